"""Host-side checks that need no GPU: the library loads, exports what include/fasted.h declares,
the dataset builders agree with the oracle and the reference's loader, the CLI rejects bad usage."""
import ctypes
import json
import os
import re
import subprocess

import numpy as np
import pytest

from conftest import GOLDEN, ROOT


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "fasted.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"typedef\s+[^;{]*\(\s*\*[^;]*;", "", text)  # function-pointer typedefs declare no symbol
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol(native_lib):
    from fasted_b200 import _lib
    declared = _declared_functions()
    assert len(declared) >= 20
    assert sorted(_lib.DECLARED_SYMBOLS) == declared
    for path in (_lib.LIB_PATH, _lib.LEGACY_LIB_PATH):
        lib = ctypes.CDLL(path)
        for name in declared:
            assert getattr(lib, name) is not None


def test_results_struct_layout_matches_reference_ctypes():
    from fasted_b200.find_pairs import Results, mmaShape
    assert ctypes.sizeof(mmaShape) == 12
    assert ctypes.sizeof(Results) == 56
    assert Results.pairsFound.offset == 16 and Results.inputProblemShape.offset == 32
    assert Results.paddedProblemShape.offset == 44


def test_selectivity_formula():
    from fasted_b200.find_pairs import compute_selectivity
    assert compute_selectivity(3000, 1000) == 2.0
    assert compute_selectivity(10, 1000) == 0


def test_no_device_is_a_loud_error(native_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from fasted_b200 import SelfJoin, FastedError
    with pytest.raises(FastedError):
        SelfJoin(0)


def test_host_generator_matches_oracle_and_reference(native_lib, oracle_mod):
    from fasted_b200 import _lib
    for pin in json.load(open(os.path.join(GOLDEN, "generator_pins.json"))):
        pts = _lib.dataset_exponential(pin["n"], pin["d"], pin["lambda"], pin["max"])
        assert np.array_equal(pts, oracle_mod.gen_exponential(pin["n"], pin["d"], pin["lambda"], pin["max"]))
        padded = np.zeros((pin["padded_n"], pin["padded_d"]), dtype=np.uint16)
        padded[: pin["n"], : pin["d"]] = pts
        assert format(oracle_mod.fnv1a64_u16(padded), "016x") == pin["fnv1a64"]


def test_host_csv_matches_reference_loader(native_lib):
    from fasted_b200 import _lib
    raw = open(os.path.join(GOLDEN, "small_csv_ref.bin"), "rb").read()
    hdr = np.frombuffer(raw[:32], dtype=np.int64)
    ref = np.frombuffer(raw[32:], dtype=np.uint16).reshape(int(hdr[0]), int(hdr[2]))
    pts = _lib.dataset_csv(os.path.join(GOLDEN, "small.csv"))
    assert pts.shape == (int(hdr[1]), int(hdr[3]))
    assert np.array_equal(ref[: pts.shape[0], : pts.shape[1]], pts)


def test_host_csv_errors(native_lib, tmp_path):
    from fasted_b200 import _lib
    ragged = tmp_path / "ragged.csv"
    ragged.write_text("1,2,3\n4,5\n")
    with pytest.raises(_lib.FastedError) as e:
        _lib.dataset_csv(str(ragged))
    assert e.value.code == _lib.EINVAL and "match the first point" in str(e.value)
    bad = tmp_path / "bad.csv"
    bad.write_text("1,2,3\n4,x,6\n")
    with pytest.raises(_lib.FastedError):
        _lib.dataset_csv(str(bad))
    empty = tmp_path / "empty.csv"
    empty.write_text("")
    with pytest.raises(_lib.FastedError):
        _lib.dataset_csv(str(empty))
    with pytest.raises(_lib.FastedError) as e:
        _lib.dataset_csv(str(tmp_path / "missing.csv"))
    assert e.value.code == _lib.EIO
    # no trailing newline, trailing delimiter, leading blanks and trailing junk are accepted like std::stod does
    ok = tmp_path / "ok.csv"
    ok.write_text("1, 2,3,\n4,5abc,6")
    pts = _lib.dataset_csv(str(ok))
    assert pts.view(np.float16).tolist() == [[1, 2, 3], [4, 5, 6]]


def test_host_half_conversion_matches_oracle(native_lib, oracle_mod, tmp_path):
    rng = np.random.default_rng(7)
    vals = np.concatenate([rng.standard_normal(4000) * 10.0 ** rng.integers(-9, 5, 4000),
                           [65504.0, 65519.0, 65520.0, 2.0 ** -24, 2.0 ** -25, 3 * 2.0 ** -25, 2.0 ** -14, 6.1e-5]])
    vals = vals[: len(vals) // 8 * 8].reshape(-1, 8)
    f = tmp_path / "v.csv"
    f.write_text("\n".join(",".join(repr(float(x)) for x in row) for row in vals) + "\n")
    from fasted_b200 import _lib
    assert np.array_equal(_lib.dataset_csv(str(f)), oracle_mod.double_to_half(vals))


def test_cli_usage_errors(native_lib):
    from fasted_b200 import _lib
    exe = os.path.join(os.path.dirname(_lib.LIB_PATH), "main")
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 1 and "Usage:" in r.stderr and "<filename> <epsilon>" in r.stderr
    r = subprocess.run([exe, "-e", "100", "64"], capture_output=True, text=True)
    assert r.returncode == 1 and "-e <numPoints> <numDimensions> <epsilon>" in r.stderr


def test_host_generator_parallel_path_is_the_same_stream(native_lib, oracle_mod):
    # Above 2^20 values the generator draws in parallel chunks (engine jump-ahead); with draws that get
    # rejected it must fall back to the sequential walk.  Both must equal the reference's stream.
    from fasted_b200 import _lib
    for n, d, lam, mx in [(1100, 1000, 40.0, 10.0), (3001, 999, 40.0, 10.0), (1500, 800, 1.0, 0.5)]:
        assert np.array_equal(_lib.dataset_exponential(n, d, lam, mx), oracle_mod.gen_exponential(n, d, lam, mx))


def test_csv_tokens_are_read_like_the_reference_reads_them(native_lib, oracle_mod, tmp_path):
    # The loader's fast number parser must agree with the std::stod the reference's loader uses
    # (source/DataLoader/FilePointGenerator.hpp of the reference), oddities and failures included;
    # the oracle's reader is the sequential restatement of that loader.
    from fasted_b200 import _lib
    p = tmp_path / "odd.csv"
    p.write_text("1e-30, +2.5,0x1p3, inf\n-0.0,1e-5 ,  3.25abc,-INF\n 4e+2,1E1,0.000000,.5\n\t7.,-.25e1,0e99,65504.9\n")
    got = _lib.dataset_csv(str(p))
    want, d = oracle_mod.read_csv(str(p))
    assert got.shape == (4, 4) and np.array_equal(got, want[:, :d])
    assert got.view(np.float16)[0].tolist() == [0.0, 2.5, 8.0, float("inf")]
    for bad in ["1,2\n3,1e-320\n", "1,2\n3,\n", "1,2\n3,abc\n", "1,2\n3,1e999\n", "1,2\n3\n"]:
        p.write_text(bad)
        with pytest.raises(_lib.FastedError):
            _lib.dataset_csv(str(p))
        with pytest.raises(RuntimeError):
            oracle_mod.read_csv(str(p))
    # a large file: same values as the sequential reader (the parallel parse splits it by lines)
    rng = np.random.default_rng(5)
    x = rng.exponential(1 / 40.0, size=(3000, 50))
    p.write_text("\n".join(",".join(f"{v:.7g}" for v in row) for row in x) + "\n")
    got = _lib.dataset_csv(str(p))
    want, d = oracle_mod.read_csv(str(p))
    assert np.array_equal(got, want[:, :d])
