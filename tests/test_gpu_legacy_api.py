"""The reference's own interface (four C entry points + CLI) on the GPU, driven the way the
reference's Python scripts and shell users drive it."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import GOLDEN, ROOT

pytestmark = pytest.mark.gpu

_DRIVER = r"""
import json, sys
sys.path.insert(0, {root!r})
from fasted_b200.find_pairs import load_findpairs, RerunnablePairsFinder
lib = load_findpairs()
out = []
finder = RerunnablePairsFinder(lambda e, s: lib.runFromExponentialDataset(1000, 64, 40.0, 10.0, e, s), lib.reRun)
for eps, save in [(0.001, False), (0.2, True), (0.001, False)]:
    r = finder(eps, save)
    out.append(dict(found=r.pairsFound, stored=r.pairsStored, tflops=r.TFLOPS, total=r.totalTime,
                    inp=[r.inputProblemShape.m, r.inputProblemShape.n, r.inputProblemShape.k],
                    pad=[r.paddedProblemShape.m, r.paddedProblemShape.n, r.paddedProblemShape.k],
                    sel=r.get_selectivity()))
r = lib.runFromFile({csv!r}.encode(), 10.0, True)
out.append(dict(found=r.pairsFound, inp=[r.inputProblemShape.m, r.inputProblemShape.n, r.inputProblemShape.k]))
lib.releaseResources()
lib.releaseResources()
print("JSON" + json.dumps(out))
"""


def test_reference_python_driver_flow(native_lib, oracle_mod, tmp_path):
    env = dict(os.environ, FASTED_OUTPUT_DIR=str(tmp_path))
    code = _DRIVER.format(root=ROOT, csv=os.path.join(GOLDEN, "small.csv"))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    out = json.loads(r.stdout.split("JSON")[-1])
    # golden: only the N self pairs at eps = 0.001 (reference's stored results for this seeded dataset)
    assert out[0]["found"] == out[0]["stored"] == 1000 and out[0]["sel"] == 0
    assert out[0]["inp"] == [1000, 1000, 64] and out[0]["pad"][2] == 64 and out[0]["pad"][0] >= 1000
    assert out[2]["found"] == 1000
    assert out[0]["tflops"] > 0 and out[0]["total"] > 0
    # reRun with a larger eps against the oracle, and the saved file in the reference's text format
    pts = oracle_mod.gen_exponential(1000, 64)
    want, _ = oracle_mod.join_fp16_fp32(pts, 0.2)
    assert abs(out[1]["found"] - len(want)) <= 4
    path = tmp_path / ("_" + f"{0.2:.6f}" + ".pairs")  # dataset name is empty on reRun, like the reference
    text = path.read_text().splitlines()
    assert len(text) == out[1]["stored"]
    got = np.array([[int(a) for a in line.split(", ")] for line in text], dtype=np.int32)
    cmp = oracle_mod.compare_pair_sets(pts, 64, 0.2, got, want, band=1e-3)
    assert cmp["ok"]
    # CSV run (5 points, one with an infinite coordinate): same count as the oracle on the same file;
    # output file named after the CSV stem
    csv_pts, csv_d = oracle_mod.read_csv(os.path.join(GOLDEN, "small.csv"))
    csv_want, _ = oracle_mod.join_fp16_fp32(csv_pts, 10.0)
    assert out[3]["found"] == len(csv_want) == 6 and out[3]["inp"] == [5, 5, 6]
    text = (tmp_path / ("small_" + f"{10.0:.6f}" + ".pairs")).read_text().splitlines()
    assert [[int(a) for a in line.split(", ")] for line in text] == csv_want.tolist()
    assert (tmp_path / ("small_" + f"{10.0:.6f}" + ".pairs")).exists()
    # the reference's stdout lines that scripts grep for
    for needle in ["Running from a generated exponential dataset", "Building point list", "Number of points is: 1000",
                   "Padded Search Dimensions:", "Input Search Dimensions:", "Number of pairs found 1000",
                   "Total Kernel Elapsed time:", "Pairs found: 1000", "Estimated TFLOPS", "Running from file: "]:
        assert needle in r.stdout, needle


def test_rerun_before_run_is_an_error(native_lib):
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from fasted_b200.find_pairs import load_findpairs\n"
            "load_findpairs().reRun(0.1, False)\n") % ROOT
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 1 and "Error: Failed to run." in r.stdout


def test_cli_synthetic_and_file(native_lib, tmp_path):
    from fasted_b200 import _lib
    exe = os.path.join(os.path.dirname(_lib.LIB_PATH), "main")
    r = subprocess.run([exe, "-e", "2154", "64", "0.001"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "Pairs found: 2154" in r.stdout and "Estimated TFLOPS" in r.stdout
    r = subprocess.run([exe, os.path.join(GOLDEN, "small.csv"), "10"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "Pairs found: 6" in r.stdout
    r = subprocess.run([exe, str(tmp_path / "nope.csv"), "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 1 and "Error: Failed to run." in r.stdout


def test_copy_points_between_contexts(gpu_join, oracle_mod):
    """Device-to-device replication used by the several-GPUs-in-one-process mode; on a one-GPU box both
    contexts sit on the same device, the call and its result are the same."""
    import torch
    from fasted_b200 import SelfJoin
    pts = oracle_mod.gen_exponential(3000, 96)
    gpu_join.set_points(pts)
    with SelfJoin(device=1 if torch.cuda.device_count() > 1 else 0) as other:
        other.copy_points_from(gpu_join)
        assert other.points_info()[1:3] == (3000, 96)
        assert np.array_equal(other.get_points(), pts.view(np.uint16))
        st = gpu_join.join(0.3, capacity=2_000_000)
        other.join(0.3, q_begin=1024, q_end=3000, capacity=2_000_000)
        want = gpu_join.pairs()
        assert st.pairs_found == st.pairs_stored > 3000
        assert np.array_equal(other.pairs(), want[want[:, 0] >= 1024])
        with pytest.raises(Exception):
            other.copy_points_from(other)


def test_broadcast_points_over_the_gpus_of_one_process(gpu_join, oracle_mod):
    """The in-library NCCL broadcast (ncclCommInitAll, one process): every further GPU receives the
    dataset of GPU 0 bit for bit and joins its band of it.  Two contexts on one GPU are refused."""
    import torch
    from fasted_b200 import SelfJoin, _lib
    pts = oracle_mod.gen_exponential(3000, 96)
    gpu_join.set_points(pts)
    with SelfJoin(0) as same:
        with pytest.raises(_lib.FastedError) as e:
            _lib.broadcast_points([gpu_join, same])
        assert e.value.code == _lib.EINVAL and "share device" in str(e.value)
    assert _lib.broadcast_points([gpu_join]) == 0.0
    g = min(torch.cuda.device_count(), 4)
    if g < 2:
        pytest.skip("needs two GPUs")
    others = [SelfJoin(i) for i in range(1, g)]
    try:
        for _ in range(2):  # the second call reuses the communicators
            ms = _lib.broadcast_points([gpu_join] + others)
            assert ms > 0
        gpu_join.join(0.3, capacity=2_000_000)
        want = gpu_join.pairs()
        for i, o in enumerate(others):
            assert o.points_info()[1:3] == (3000, 96)
            assert np.array_equal(o.get_points(), pts.view(np.uint16))
            o.join(0.3, q_begin=1024 * (i % 2), q_end=3000, capacity=2_000_000)
            assert np.array_equal(o.pairs(), want[want[:, 0] >= 1024 * (i % 2)])
    finally:
        for o in others:
            o.close()


_TWO_GPU_DRIVER = r"""
import sys
sys.path.insert(0, {root!r})
from fasted_b200.find_pairs import load_findpairs
lib = load_findpairs()
r = lib.runFromExponentialDataset(5000, 200, 40.0, 10.0, 0.36, True)
r2 = lib.reRun(0.3, False)
assert r.pairsFound == r.pairsStored > 5000
lib.releaseResources()
print("COUNTS", r.pairsFound, r.pairsStored, r2.pairsFound)
"""


def test_one_process_two_gpus_writes_the_same_file(native_lib, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    seen = []
    for gpus, sym in (("1", "1"), ("2", "1"), ("all", "1"), ("2", "0")):
        out = tmp_path / (gpus + sym)
        out.mkdir()
        env = dict(os.environ, FASTED_OUTPUT_DIR=str(out) + "/", FASTED_NUM_GPUS=gpus, FASTED_WRITE_DIST="1",
                   FASTED_SYMMETRIC=sym)
        r = subprocess.run([sys.executable, "-c", _TWO_GPU_DRIVER.format(root=ROOT)], capture_output=True, text=True,
                           env=env, timeout=600)
        assert r.returncode == 0, r.stdout + r.stderr
        files = list(out.iterdir())
        assert len(files) == 1
        seen.append((files[0].read_text(), [l for l in r.stdout.splitlines() if l.startswith("COUNTS")]))
    assert len(seen[0][0].splitlines()) > 5000
    assert seen[0] == seen[1] == seen[2] == seen[3]


def test_more_gpus_than_present_is_an_error(native_lib):
    from fasted_b200 import _lib
    exe = os.path.join(os.path.dirname(_lib.LIB_PATH), "main")
    env = dict(os.environ, FASTED_NUM_GPUS="64")
    r = subprocess.run([exe, "-e", "1000", "64", "0.1"], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 1 and "Error: Failed to run." in r.stdout


_REFERENCE_DRIVER = r"""
import json, os, sys
sys.path.insert(0, os.path.join({ref!r}, "results", "scripts"))
from experiment.find_pairs import load_findpairs, RerunnablePairsFinder     # the reference's own modules,
from experiment.experiments import ExperimentRunner, SearchParameters, find_epsilon_binary, bound_epsilon
lib = load_findpairs()                      # loads ../../source/main.so relative to the working directory
runner = ExperimentRunner(lib)
finder = RerunnablePairsFinder(lambda e, s: lib.runFromExponentialDataset(10000, 64, 40.0, 10.0, e, s), lib.reRun)
sel = lambda eps: finder(eps, False).get_selectivity()
lo, hi = bound_epsilon(0.01, 100000, 16.0, sel)
eps = find_epsilon_binary(16.0, sel, initial_epsilon=0.01)
trials = runner.run_time_trials(finder, [SearchParameters(16.0, eps, False)], 3)
lib.releaseResources()
print("JSON" + json.dumps(dict(lo=lo, hi=hi, eps=eps, sel=[t.results.get_selectivity() for t in trials],
                               found=[t.results.pairsFound for t in trials], tflops=[t.results.TFLOPS for t in trials])))
"""


def test_the_references_own_driver_runs_against_this_library(native_lib, oracle_mod, tmp_path):
    """The reference's experiment driver itself (results/scripts/experiment: load_findpairs, bound_epsilon,
    find_epsilon_binary, run_time_trials), unmodified, with this library in the place of its main.so.
    Needs the reference checkout (environment variable FASTED_REFERENCE_ROOT); skipped without it."""
    from fasted_b200 import _lib
    ref = os.environ.get("FASTED_REFERENCE_ROOT", "/root/reference")
    if not os.path.isdir(os.path.join(ref, "results", "scripts", "experiment")):
        pytest.skip("the reference checkout is not present on this machine")
    (tmp_path / "source").mkdir()
    os.symlink(_lib.LEGACY_LIB_PATH, tmp_path / "source" / "main.so")
    cwd = tmp_path / "results" / "scripts"
    cwd.mkdir(parents=True)
    r = subprocess.run([sys.executable, "-c", _REFERENCE_DRIVER.format(ref=ref)], capture_output=True, text=True,
                       cwd=str(cwd), env=dict(os.environ, FASTED_OUTPUT_DIR=str(tmp_path)), timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    out = json.loads(r.stdout.split("JSON")[-1])
    assert out["lo"] < out["eps"] < out["hi"]
    assert all(abs(s - 16.0) <= 0.16 + 1e-9 for s in out["sel"])  # within a percent of the target, as the driver asks
    assert len(set(out["found"])) == 1 and all(t > 0 for t in out["tflops"])
    # the count the driver converged on is the oracle's count at that epsilon
    pts = oracle_mod.gen_exponential(10000, 64)
    want, _ = oracle_mod.join_fp16_fp32(pts, out["eps"])
    assert out["found"][0] == len(want)
