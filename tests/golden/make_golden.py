"""Regenerates the CPU-side golden fixtures in this directory.

Run in the build container, where the reference checkout is mounted:

    make -C oracle ref            # compiles the reference's loader headers -> oracle/_ref/ref_datagen
    python tests/golden/make_golden.py [reference_root]

What is produced, and from what:

  generator_pins.json   output of the reference's own ExponentialPointGenerator +
                        PointListBuilder<half> (oracle/_ref/ref_datagen): padded shape, first 8
                        binary16 patterns, FNV-1a-64 over all binary16 patterns.
  small.csv, small_csv_ref.bin
                        a hand-made CSV that exercises the parser, and the reference loader's
                        binary16 output for it.
  selfpair_counts.json  (N, D, epsilon, pairsFound) rows with D <= 256 copied from the reference's
                        stored benchmark results for its seeded synthetic mode
                        (results/speed_results/ExpoDataSpeedVsSize_OnDemandRasterizer.json).
  config1_fp64.json     FP64 brute-force result (oracle) on the 4096 x 128 synthetic dataset.

The GPU-side fixtures (ref_gpu_*.npz) come from make_golden_gpu.py, which needs a B200.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

REF = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
DATAGEN = os.path.join(ROOT, "oracle", "_ref", "ref_datagen")


def read_bin(path):
    raw = open(path, "rb").read()
    hdr = np.frombuffer(raw[:32], dtype=np.int64)
    vals = np.frombuffer(raw[32:], dtype=np.uint16).reshape(int(hdr[0]), int(hdr[2]))
    return [int(x) for x in hdr], vals


def generator_pins():
    pins = []
    with tempfile.TemporaryDirectory() as tmp:
        for n, d, dim_factor, pts_factor in [(1000, 64, 64, 768), (4096, 128, 64, 64), (333, 100, 64, 768), (50, 7, 64, 8)]:
            out = os.path.join(tmp, "o.bin")
            subprocess.check_call([DATAGEN, "exp", str(n), str(d), "40", "10.0", str(dim_factor), str(pts_factor), out],
                                  stdout=subprocess.DEVNULL)
            hdr, vals = read_bin(out)
            pins.append({
                "n": n, "d": d, "lambda": 40.0, "max": 10.0, "dim_factor": dim_factor, "points_factor": pts_factor,
                "padded_n": hdr[0], "padded_d": hdr[2],
                "first8": [int(x) for x in vals.reshape(-1)[:8]],
                "fnv1a64": format(oracle.fnv1a64_u16(vals), "016x"),
            })
    json.dump(pins, open(os.path.join(HERE, "generator_pins.json"), "w"), indent=1)


def small_csv():
    rows = [
        "0.5,1.25,-3.0, 7e-3,65504,1e-8",
        "  2.5,0.333333333,1e5,-1e-5,5.9604645e-8,0.1",
        "1,2,3,4,5,6",
        "0.0999755859375,0.099975586,0.09997559,2049,2051,-0",
        "3.0000001,6.1e-5,6.0e-5,1e-7,2.98e-8,2.99e-8",
    ]
    path = os.path.join(HERE, "small.csv")
    open(path, "w").write("\n".join(rows) + "\n")
    out = os.path.join(HERE, "small_csv_ref.bin")
    subprocess.check_call([DATAGEN, "csv", path, "64", "8", out], stdout=subprocess.DEVNULL)


def selfpair_counts():
    src = os.path.join(REF, "results", "speed_results", "ExpoDataSpeedVsSize_OnDemandRasterizer.json")
    rows = {}
    for e in json.load(open(src)):
        r = e["results"]
        n, d = r["inputProblemShape"]["m"], r["inputProblemShape"]["k"]
        if d <= 256 and n <= 100000:
            rows[(n, d)] = {"n": n, "d": d, "epsilon": e["epsilon"], "pairsFound": r["pairsFound"]}
    json.dump(sorted(rows.values(), key=lambda x: (x["d"], x["n"])),
              open(os.path.join(HERE, "selfpair_counts.json"), "w"), indent=1)


def config1():
    pts = oracle.gen_exponential(4096, 128)
    eps = 0.3136
    pairs, d2, found = oracle.join_fp64(pts, eps)
    keys = oracle.pair_keys(pairs)
    eps2 = eps * eps
    json.dump({
        "n": 4096, "d": 128, "epsilon": eps, "pairs_fp64": int(found),
        "pairs_in_band_1e-3": int(np.sum(np.abs(d2 - eps2) <= 1e-3 * eps2)),
        "key_sum_mod_2_64": int(np.sum(keys, dtype=np.uint64)),
        "dataset_fnv1a64": format(oracle.fnv1a64_u16(pts), "016x"),
    }, open(os.path.join(HERE, "config1_fp64.json"), "w"), indent=1)


if __name__ == "__main__":
    generator_pins()
    small_csv()
    selfpair_counts()
    config1()
    print("golden fixtures written to", HERE)
