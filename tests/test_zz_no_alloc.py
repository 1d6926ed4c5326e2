"""fasted_join_static_scratch, the entry point for callers that must not allocate (hosts that own
the whole GPU memory pool, callers that cannot afford the device-wide stall of cudaMalloc).

Collected last on purpose.  It calls the entry point through the C ABI on buffers that the test
allocates itself (standing in for the host's pool), twice in a row with different inputs, and
compares each result with fasted_join on the same input: same pair set bit for bit, since both
run the same kernels (the tolerance band of the other parity tests is not needed here)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run_case(oracle_mod, sj, pts, d, eps, capacity=None):
    import torch
    from fasted_b200 import _lib
    n, ld = pts.shape
    dev = torch.from_numpy(pts.view(np.int16)).cuda()
    want_sj = sj
    want_sj.set_points(pts, d)
    st = want_sj.join(eps, capacity=capacity or 0)
    want = want_sj.pairs()
    cap = capacity or max(1, int(st.pairs_found))
    out = torch.full((cap,), -1, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    found, stored = _lib.join_static_scratch(dev.data_ptr(), n, d, ld, eps, out.data_ptr(), cap)
    keys = np.sort(out.cpu().numpy().view(np.uint64)[:stored])
    assert found == st.pairs_found and stored == min(found, cap)
    if capacity is None:
        assert stored == found == len(want)
        assert np.array_equal(keys, oracle_mod.pair_keys(want))
    else:
        # overflow: what was stored is a duplicate-free subset of the full result
        full_sj = sj.join(eps)
        allk = oracle_mod.pair_keys(sj.pairs())
        assert len(np.unique(keys)) == stored and np.isin(keys, allk).all()
    return found


def test_static_scratch_join_matches_fasted_join_twice(gpu_join, oracle_mod):
    # call 1: larger n and d (fills more of the scratch area) ...
    a = oracle_mod.gen_exponential(3000, 192)
    fa = _run_case(oracle_mod, gpu_join, a, 192, 0.36)
    # ... call 2 right after it: fewer points, other epsilon; must not see call 1's counters or norms
    rng = np.random.default_rng(11)
    b = np.zeros((777, 72), dtype=np.uint16)  # d = 70 inside a row stride of 72 (multiple of 8), zero padded
    b[:, :70] = oracle_mod.double_to_half(rng.exponential(1 / 40.0, size=(777, 70)))
    fb = _run_case(oracle_mod, gpu_join, b, 70, 0.21)
    assert fa > 3000 and fb > 777
    # and against the CPU oracle once, within the band the other parity tests use
    import torch
    from fasted_b200 import _lib
    dev = torch.from_numpy(b.view(np.int16)).cuda()
    out = torch.zeros((fb,), dtype=torch.int64, device="cuda")
    found, stored = _lib.join_static_scratch(dev.data_ptr(), 777, 70, 72, 0.21, out.data_ptr(), fb)
    k = np.sort(out.cpu().numpy().view(np.uint64))
    got = np.stack([(k >> np.uint64(32)).astype(np.int32), (k & np.uint64(0xFFFFFFFF)).astype(np.int32)], 1)
    want, _ = oracle_mod.join_fp16_fp32(np.ascontiguousarray(b[:, :70]), 0.21)
    assert oracle_mod.compare_pair_sets(np.ascontiguousarray(b[:, :70]), 70, 0.21, got, want, band=1e-3)["ok"]


def test_static_scratch_overflow_and_limits(gpu_join, oracle_mod):
    from fasted_b200 import _lib
    pts = oracle_mod.gen_exponential(600, 64)
    _run_case(oracle_mod, gpu_join, pts, 64, 0.25, capacity=1000)
    import torch
    dev = torch.zeros((8, 64), dtype=torch.float16, device="cuda")
    out = torch.zeros((8,), dtype=torch.int64, device="cuda")
    with pytest.raises(_lib.FastedError) as e:  # beyond the built-in scratch area: refused, nothing launched
        _lib.join_static_scratch(dev.data_ptr(), (1 << 20) + 1, 64, 64, 0.1, out.data_ptr(), 8)
    assert e.value.code == _lib.EINVAL and "exceeds" in str(e.value)
    with pytest.raises(_lib.FastedError):
        _lib.join_static_scratch(dev.data_ptr(), 8, 64, 60, 0.1, out.data_ptr(), 8)  # bad row stride
    # count-only use: no output buffer at all
    found, stored = _lib.join_static_scratch(dev.data_ptr(), 8, 64, 64, 0.0, 0, 0)
    assert found == 64 and stored == 0


def test_static_scratch_leaves_free_memory_alone(gpu_join, oracle_mod):
    """The property in the entry point's name: once the library's module is on the GPU, a call changes
    nothing about the amount of free device memory (no cudaMalloc / cudaFree hides inside it)."""
    import torch
    from fasted_b200 import _lib
    pts = oracle_mod.gen_exponential(2000, 128)
    dev = torch.from_numpy(pts.view(np.int16)).cuda()
    out = torch.zeros((1 << 20,), dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    first = _lib.join_static_scratch(dev.data_ptr(), 2000, 128, 128, 0.3, out.data_ptr(), 1 << 20)
    free_before, _ = torch.cuda.mem_get_info()
    second = _lib.join_static_scratch(dev.data_ptr(), 2000, 128, 128, 0.3, out.data_ptr(), 1 << 20)
    third = _lib.join_static_scratch(dev.data_ptr(), 1500, 128, 128, 0.25, out.data_ptr(), 1 << 20)
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert first == second and third[0] < second[0]


_FIRST_CALL = r"""
import sys
sys.path.insert(0, {root!r})
import numpy as np, torch
import oracle
from fasted_b200 import _lib, SelfJoin
pts = oracle.gen_exponential(1500, 96)
dev = torch.from_numpy(pts.view(np.int16)).cuda()          # the host's pool stands in: torch owns these
out = torch.zeros((1 << 19,), dtype=torch.int64, device="cuda")
torch.cuda.synchronize()
# The very first call into the library in this process: it is the one that makes the CUDA runtime
# load the library's module (kernels + the built-in scratch area) on this GPU.
free0, _ = torch.cuda.mem_get_info()
found1, stored1 = _lib.join_static_scratch(dev.data_ptr(), 1500, 96, 96, 0.3, out.data_ptr(), 1 << 19)
free1, _ = torch.cuda.mem_get_info()
k1 = np.sort(out.cpu().numpy().view(np.uint64)[:stored1])
found2, stored2 = _lib.join_static_scratch(dev.data_ptr(), 1500, 96, 96, 0.3, out.data_ptr(), 1 << 19)
free2, _ = torch.cuda.mem_get_info()
k2 = np.sort(out.cpu().numpy().view(np.uint64)[:stored2])
with SelfJoin(0) as sj:                                      # the allocating entry point, for comparison
    sj.set_points(pts)
    st = sj.join(0.3)
    want = oracle.pair_keys(sj.pairs())
assert found1 == found2 == st.pairs_found == len(want), (found1, found2, st.pairs_found)
assert np.array_equal(k1, want) and np.array_equal(k2, want)
assert free2 == free1, (free1, free2)                        # later calls take nothing
print("MODULE_LOAD_BYTES", free0 - free1)
"""


def test_static_scratch_as_the_first_call_of_a_process(native_lib, oracle_mod):
    """In a fresh process the entry point is the first thing asked of the library, so this call is the
    one during which the CUDA runtime places the library's module on the GPU; it must work, give the
    allocating entry point's result, and every call after it must leave free memory untouched."""
    import subprocess
    import sys
    from conftest import ROOT
    r = subprocess.run([sys.executable, "-c", _FIRST_CALL.format(root=ROOT)], capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "MODULE_LOAD_BYTES" in r.stdout
