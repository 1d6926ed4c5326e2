"""Shared checks for the GPU parity tests."""
import numpy as np


def assert_pairs_match(oracle_mod, pts, d, eps, got_pairs, want_pairs, band=1e-3, what=""):
    """Pair sets must be identical except for pairs whose FP64 squared distance lies within
    band * eps^2 of eps^2 (the tolerance the task states for this FP16->FP32 path)."""
    cmp = oracle_mod.compare_pair_sets(pts, d, eps, got_pairs, want_pairs, band=band)
    assert cmp["ok"], (f"{what}: {len(cmp['unexcused_a'])} pairs only in ours, {len(cmp['unexcused_b'])} only in "
                       f"the oracle's, outside the band; first: {cmp['unexcused_a'][:3]} {cmp['unexcused_b'][:3]} "
                       f"(sizes {cmp['n_a']} / {cmp['n_b']})")
    return cmp


def assert_sorted_unique(oracle_mod, pairs):
    keys = oracle_mod.pair_keys(pairs).astype(np.int64)
    assert (np.diff(keys) > 0).all(), "pairs are not in strict row-major order"


def assert_dist_close(oracle_mod, pts, d, pairs, d2, rtol=1e-3):
    """Emitted FP32 squared distances vs FP64, 1e-3 relative (absolute floor for the diagonal)."""
    if len(pairs) == 0:
        return
    want = oracle_mod.pair_d2_fp64(pts, pairs, d)
    norms = oracle_mod.row_norms(pts, d).astype(np.float64)
    scale = norms[pairs[:, 0]] + norms[pairs[:, 1]]
    err = np.abs(d2.astype(np.float64) - want)
    # d2 is a difference of numbers of size `scale`, so FP32 noise is relative to `scale` whatever d2
    # is (the diagonal has d2 = 0 exactly in FP64).  The reference's row norms are a chain of d/2
    # round-toward-zero adds, each losing up to one ulp of the running sum: about d/8 ulps in all.
    floor = max(4e-6, d / 8 * 2.0 ** -23) * scale
    assert (err <= rtol * want + floor).all(), float(np.max(err / (rtol * want + floor)))


def assert_identical_to_oracle(oracle_mod, pts, d, eps, got_pairs, got_d2=None, q_begin=0, q_end=None):
    """The CPU oracle models the B200's tensor-core accumulate bit for bit, so the CUDA path must give
    exactly the oracle's pairs (and, when recorded, exactly its FP32 squared distances)."""
    want, want_d2 = oracle_mod.join_fp16_fp32(pts, eps, d=d, q_begin=q_begin, q_end=q_end)
    assert np.array_equal(got_pairs, want), (len(got_pairs), len(want))
    if got_d2 is not None:
        assert np.array_equal(got_d2.view(np.uint32), want_d2.view(np.uint32))
    return want
