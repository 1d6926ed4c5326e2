"""Builds the native library in-tree with nvcc for sm_100a.

    python -m fasted_b200.build            # libfasted.so, main.so (same file), main

Outputs land in fasted_b200/lib/ (git-ignored, shipped as built files).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
HOST_CXX = "/usr/bin/g++"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-I", os.path.join(ROOT, "include"), "-I", CSRC,
          "-ccbin", HOST_CXX, "-Xcompiler", "-fPIC,-fopenmp,-Wall,-Wno-unknown-pragmas"]

LIB_SOURCES = ["fasted.cu", "dataset.cpp", "dataset_api.cpp", "legacy_api.cpp"]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    lib = os.path.join(LIBDIR, "libfasted.so")
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "fasted.h"), __file__]
    if force or _stale(lib, deps):
        cmd = [NVCC, *ARCH, *COMMON, "-shared", "-o", lib, *[os.path.join(CSRC, s) for s in LIB_SOURCES],
               "-Xptxas", "-v" if verbose else "-warn-spills", "-lgomp", "-ldl"]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    # The reference's Python driver loads "main.so"; ship the same library under that name.
    alias = os.path.join(LIBDIR, "main.so")
    if force or _stale(alias, [lib]):
        shutil.copyfile(lib, alias)
    exe = os.path.join(LIBDIR, "main")
    if force or _stale(exe, [lib, os.path.join(CSRC, "main.cpp")]):
        subprocess.check_call([HOST_CXX, "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"),
                               os.path.join(CSRC, "main.cpp"), "-o", exe, "-L", LIBDIR, "-lfasted",
                               "-Wl,-rpath,$ORIGIN"])
    return lib


if __name__ == "__main__":
    build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(os.path.join(LIBDIR, "libfasted.so"))
