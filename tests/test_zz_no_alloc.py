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
