"""The join through the C ABI vs the CPU oracle on the same inputs.

Bar stated for this FP16 -> FP32 path: pair sets identical except for pairs whose FP64 squared distance
lies within 1e-3 * eps^2 of eps^2; emitted squared distances within 1e-3 relative.  What is asserted
is stronger wherever the oracle runs: the oracle models the B200's tensor-core accumulate bit for bit
(see test_raw_accumulators_match_the_accumulate_model), so pairs and FP32 distances must be IDENTICAL
to it; the band and the tolerance are only used against FP64 truth."""
import json
import os

import numpy as np
import pytest

from conftest import GOLDEN
from util import assert_dist_close, assert_identical_to_oracle, assert_pairs_match, assert_sorted_unique

pytestmark = pytest.mark.gpu

BAND = 1e-3


def _eps_for_mean_neighbours(oracle_mod, pts, target):
    """Epsilon giving about `target` neighbours per point, from FP64 distances of a row sample."""
    f = pts.view(np.float16).astype(np.float64)
    rows = f[: max(8, len(f) // 100)]
    d2 = ((rows ** 2).sum(1)[:, None] + (f ** 2).sum(1)[None, :] - 2 * rows @ f.T).ravel()
    q = min(1.0, (target + 1) / len(f))
    return float(np.sqrt(max(np.quantile(d2, q), 1e-12)))


@pytest.mark.parametrize("n,d,target", [
    (64, 64, 4), (128, 64, 8), (256, 128, 8), (257, 64, 8), (300, 100, 8), (1000, 64, 16),
    (1024, 192, 16), (777, 333, 8), (2048, 128, 32), (520, 1024, 8),
])
def test_join_matches_oracle_small(gpu_join, oracle_mod, n, d, target):
    rng = np.random.default_rng(n * 31 + d)
    pts = oracle_mod.double_to_half(rng.exponential(1 / 40.0, size=(n, d)))
    eps = _eps_for_mean_neighbours(oracle_mod, pts, target)
    gpu_join.set_points(pts)
    st = gpu_join.join(eps, flags=1)
    got, d2 = gpu_join.pairs(with_dist2=True)
    assert st.status == 0 and st.pairs_found == st.pairs_stored == len(got)
    assert_sorted_unique(oracle_mod, got)
    want = assert_identical_to_oracle(oracle_mod, pts, d, eps, got, d2)
    assert_pairs_match(oracle_mod, pts, d, eps, got, oracle_mod.join_fp64(pts, eps)[0], BAND, f"{n}x{d} vs FP64")
    assert_dist_close(oracle_mod, pts, d, got, d2)
    # every real point pairs with itself at these epsilons, nothing refers to padding
    assert got.min() >= 0 and got.max() < n
    assert np.isin(oracle_mod.pair_keys(np.stack([np.arange(n)] * 2, 1)), oracle_mod.pair_keys(got)).all()


def test_join_config1_reference_dataset(gpu_join, oracle_mod):
    # 4096 x 128 seeded synthetic dataset, eps for ~32 neighbours per point.
    g = json.load(open(os.path.join(GOLDEN, "config1_fp64.json")))
    pts = oracle_mod.gen_exponential(g["n"], g["d"])
    gpu_join.set_points(pts)
    st = gpu_join.join(g["epsilon"], flags=1)
    got, d2 = gpu_join.pairs(with_dist2=True)
    assert_identical_to_oracle(oracle_mod, pts, g["d"], g["epsilon"], got, d2)
    want64, _, found64 = oracle_mod.join_fp64(pts, g["epsilon"])
    assert found64 == g["pairs_fp64"]
    cmp64 = assert_pairs_match(oracle_mod, pts, g["d"], g["epsilon"], got, want64, BAND, "vs FP64")
    assert cmp64["only_a"] + cmp64["only_b"] <= 64
    assert abs(int(st.pairs_found) - g["pairs_fp64"]) <= 64
    assert_dist_close(oracle_mod, pts, g["d"], got, d2)


@pytest.mark.parametrize("idx", range(4))
def test_join_selfpair_goldens(gpu_join, oracle_mod, idx):
    # The reference's stored results for its seeded synthetic mode at eps = 0.001: pairsFound == N.
    rows = [r for r in json.load(open(os.path.join(GOLDEN, "selfpair_counts.json"))) if r["n"] <= 21544]
    rows = sorted(rows, key=lambda r: (r["n"], r["d"]))[::3][:4]
    r = rows[idx]
    pts = oracle_mod.gen_exponential(r["n"], r["d"])
    gpu_join.set_points(pts)
    st = gpu_join.join(r["epsilon"])
    got = gpu_join.pairs()
    assert st.pairs_found == r["pairsFound"]
    assert np.array_equal(got[:, 0], np.arange(r["n"])) and np.array_equal(got[:, 1], np.arange(r["n"]))


def test_join_unit_vectors_gaussian(gpu_join, oracle_mod):
    # Shape family of the mid-size config: N(0,1) rows normalised to unit length.
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3000, 384)).astype(np.float32)
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    pts = oracle_mod.double_to_half(x.astype(np.float64))
    eps = _eps_for_mean_neighbours(oracle_mod, pts, 16)
    gpu_join.set_points(pts)
    gpu_join.join(eps, flags=1)
    got, d2 = gpu_join.pairs(with_dist2=True)
    assert_identical_to_oracle(oracle_mod, pts, 384, eps, got, d2)
    assert_dist_close(oracle_mod, pts, 384, got, d2)


def test_join_dense_clusters(gpu_join, oracle_mod):
    # Output-heavy case: tight clusters, most entries of a tile hit.
    rng = np.random.default_rng(5)
    centres = rng.uniform(0, 1, size=(6, 96))
    which = rng.integers(0, 6, size=1500)
    pts = oracle_mod.double_to_half(centres[which] + rng.normal(0, 0.05, size=(1500, 96)))
    eps = 0.9
    gpu_join.set_points(pts)
    st = gpu_join.join(eps)
    got = gpu_join.pairs()
    assert st.pairs_found > 200_000
    assert_sorted_unique(oracle_mod, got)
    assert_identical_to_oracle(oracle_mod, pts, 96, eps, got)


def test_join_edge_epsilons(gpu_join, oracle_mod):
    pts = oracle_mod.gen_exponential(500, 64)
    gpu_join.set_points(pts)
    # eps = 0: d2(i,i) is exactly 0 only when s_i + s_i == 2 a_ii bit for bit; compare with >= nothing else
    st = gpu_join.join(0.0)
    got = gpu_join.pairs()
    assert (got[:, 0] == got[:, 1]).all() or len(got) == 0
    # huge eps: everything pairs, padding never does
    st = gpu_join.join(1e3, capacity=500 * 500)
    assert st.pairs_found == st.pairs_stored == 500 * 500
    got = gpu_join.pairs()
    assert np.array_equal(oracle_mod.pair_keys(got),
                          oracle_mod.pair_keys(np.stack(np.meshgrid(np.arange(500), np.arange(500), indexing="ij"), -1).reshape(-1, 2)))
    # identical points: all-zero rows pair with each other at eps 0
    z = np.zeros((130, 64), dtype=np.uint16)
    gpu_join.set_points(z)
    assert gpu_join.join(0.0).pairs_found == 130 * 130
    # default capacity is the reference's n * 256 rule: 500 * 500 pairs do not fit 500 * 256 slots
    gpu_join.set_points(pts)
    st = gpu_join.join(1e3)
    assert st.pairs_found == 500 * 500 and st.pairs_stored == 500 * 256


def test_join_overflow_semantics(gpu_join, oracle_mod):
    # Pair buffer too small: found keeps counting, stored saturates at the capacity
    # (source/pair.cuh:123-133 of the reference).
    pts = oracle_mod.gen_exponential(600, 64)
    gpu_join.set_points(pts)
    full = gpu_join.join(0.25)
    assert full.pairs_found == full.pairs_stored > 5000
    st = gpu_join.join(0.25, capacity=1000)
    assert st.pairs_found == full.pairs_found and st.pairs_stored == 1000
    got = gpu_join.pairs()
    assert len(got) == 1000
    gpu_join.join(0.25)
    allp = oracle_mod.pair_keys(gpu_join.pairs())
    assert np.isin(oracle_mod.pair_keys(got), allp).all() and len(np.unique(oracle_mod.pair_keys(got))) == 1000


def test_join_bands_concatenate(gpu_join, oracle_mod):
    # Query-row bands (the multi-GPU sharding unit): concatenation in band order == full join.
    pts = oracle_mod.gen_exponential(1500, 128)
    gpu_join.set_points(pts)
    eps = 0.3
    gpu_join.join(eps)
    full = gpu_join.pairs()
    parts = []
    for a, b in [(0, 384), (384, 385), (385, 1000), (1000, 1500)]:
        gpu_join.join(eps, q_begin=a, q_end=b)
        p = gpu_join.pairs()
        assert len(p) == 0 or (p[:, 0].min() >= a and p[:, 0].max() < b)
        parts.append(p)
    assert np.array_equal(np.concatenate(parts), full)
    st = gpu_join.join(eps, q_begin=700, q_end=700)
    assert st.pairs_found == 0


def test_join_rerun_is_idempotent_and_monotone(gpu_join, oracle_mod):
    pts = oracle_mod.gen_exponential(2000, 64)
    gpu_join.set_points(pts)
    a = gpu_join.join(0.2)
    pa = gpu_join.pairs()
    b = gpu_join.join(0.2, flags=4)  # keep norms
    pb = gpu_join.pairs()
    assert a.pairs_found == b.pairs_found and np.array_equal(pa, pb)
    c = gpu_join.join(0.22)
    assert c.pairs_found >= a.pairs_found
    assert np.isin(oracle_mod.pair_keys(pa), oracle_mod.pair_keys(gpu_join.pairs())).all()


def test_join_device_pointer_input(gpu_join, oracle_mod):
    import torch
    pts = oracle_mod.gen_exponential(900, 128)
    gpu_join.set_points(pts)
    gpu_join.join(0.3)
    want = gpu_join.pairs()
    t = torch.from_numpy(pts.view(np.int16)).cuda()
    gpu_join.set_points_device(t.data_ptr(), 900, 128, 128, keepalive=t)
    gpu_join.join(0.3)
    assert np.array_equal(gpu_join.pairs(), want)


def test_join_argument_errors(gpu_join, oracle_mod):
    from fasted_b200 import FastedError
    pts = oracle_mod.gen_exponential(100, 64)
    gpu_join.set_points(pts)
    with pytest.raises(FastedError):
        gpu_join.join(0.1, q_begin=50, q_end=200)
    with pytest.raises(FastedError):
        gpu_join.join(float("nan"))
    # only eps^2 enters the test, as in the reference: a negative epsilon equals its absolute value
    a = gpu_join.join(0.3).pairs_found
    assert gpu_join.join(-0.3).pairs_found == a
    with pytest.raises(FastedError):
        gpu_join.set_points(np.zeros((0, 64), dtype=np.uint16))


def test_join_midsize_properties(gpu_join, oracle_mod):
    # Larger than the oracle can brute-force quickly: size-independent properties.
    n, d = 40_000, 256
    gpu_join.generate_exponential(n, d)
    pts = gpu_join.get_points()
    eps = _eps_for_mean_neighbours(oracle_mod, pts, 16)
    st = gpu_join.join(eps, flags=1)
    got, d2 = gpu_join.pairs(with_dist2=True)
    assert st.pairs_found == st.pairs_stored == len(got)
    assert_sorted_unique(oracle_mod, got)
    keys = oracle_mod.pair_keys(got)
    # symmetry and the diagonal
    assert np.array_equal(np.sort(oracle_mod.pair_keys(got[:, ::-1])), keys)
    assert np.isin(oracle_mod.pair_keys(np.stack([np.arange(n)] * 2, 1)), keys).all()
    # every emitted pair is a true neighbour up to the band, distances agree with FP64
    true_d2 = oracle_mod.pair_d2_fp64(pts, got, d)
    assert (true_d2 <= eps * eps * (1 + BAND)).all()
    assert_dist_close(oracle_mod, pts, d, got, d2)
    # completeness on sampled rows, against both the CPU FP64 join and the device FP64 check
    rows = np.arange(0, n, n // 64)[:64]
    counts_dev = gpu_join.brute_force_counts(rows, eps)
    for i, r in enumerate(rows[:8]):
        want, _, _ = oracle_mod.join_fp64(pts, eps, q_begin=int(r), q_end=int(r) + 1)
        mine = got[got[:, 0] == r]
        assert_pairs_match(oracle_mod, pts, d, eps, mine, want, BAND, f"row {r}")
        assert abs(int(counts_dev[i]) - len(want)) == 0
    per_row = np.bincount(got[:, 0], minlength=n)[rows]
    assert np.abs(per_row.astype(np.int64) - counts_dev.astype(np.int64)).max() <= 2


def _ref_gpu_cases():
    import glob
    return sorted(glob.glob(os.path.join(GOLDEN, "ref_gpu_*.npz")))


@pytest.mark.parametrize("path", _ref_gpu_cases(), ids=lambda p: os.path.basename(p)[8:-4])
def test_join_against_reference_gpu_output(gpu_join, oracle_mod, path):
    # Same inputs as the reference's own kernels were run on (fixtures recorded on a B200).
    from test_oracle_golden import _golden_dataset
    g = np.load(path)
    pts = _golden_dataset(oracle_mod, g)
    eps, d = float(g["epsilon"]), int(g["d"])
    gpu_join.set_points(pts)
    st = gpu_join.join(eps)
    got = gpu_join.pairs()
    # On a B200 the reference's mma.sync kernels and this library's tcgen05 kernels accumulate alike:
    # the outputs are identical, pair for pair (the band is not needed here).
    assert int(st.pairs_found) == int(g["pairs_found"])
    assert np.array_equal(got, g["pairs"])


@pytest.mark.parametrize("n,d,eps", [(256, 64, 1e3), (300, 100, 1e3), (1000, 256, 0.5), (2000, 512, 0.7), (5000, 448, 0.68),
                                     (4096, 128, 0.3136), (777, 333, 0.62), (20_000, 384, 0.58), (9000, 64, 0.2),
                                     (1, 8, 1.0), (130, 512, 1e3)])
def test_query_stationary_kernel_is_bit_identical(gpu_join, oracle_mod, n, d, eps):
    # Short rows can be joined by the kernel that keeps a CTA's query tile in shared memory and walks
    # tile rows instead of raster bands.  Same accumulators, same K order: pairs and distances must
    # equal the raster kernel's bit for bit, for the full and the symmetric schedule, bands included.
    rng = np.random.default_rng(7 * n + d)
    pts = oracle_mod.double_to_half(rng.exponential(1 / 40.0, size=(n, d)))
    gpu_join.set_points(pts)
    try:
        gpu_join.set_option("query_stationary", 0)
        a = gpu_join.join(eps, capacity=min(n * n, 40_000_000), flags=1)
        pa, da = gpu_join.pairs(with_dist2=True)
        gpu_join.set_option("query_stationary", 1)
        b = gpu_join.join(eps, capacity=min(n * n, 40_000_000), flags=1)
        pb, db = gpu_join.pairs(with_dist2=True)
        assert a.status == 0 and b.status == 0 and a.pairs_found == b.pairs_found == len(pa)
        assert np.array_equal(pa, pb) and np.array_equal(da.view(np.uint32), db.view(np.uint32))
        c = gpu_join.join(eps, capacity=min(n * n, 40_000_000), flags=1 | 8)
        pc, dc = gpu_join.pairs(with_dist2=True)
        assert c.pairs_found == a.pairs_found
        assert np.array_equal(pa, pc) and np.array_equal(da.view(np.uint32), dc.view(np.uint32))
        if n > 600:
            gpu_join.join(eps, q_begin=128, q_end=min(n, 600), capacity=min(n * n, 40_000_000))
            assert np.array_equal(gpu_join.pairs(), pa[(pa[:, 0] >= 128) & (pa[:, 0] < min(n, 600))])
            st = gpu_join.join_stream(eps, capacity=min(n * n, 40_000_000))
            assert st.pairs_found == a.pairs_found and np.array_equal(gpu_join.pairs(), pa)
    finally:
        gpu_join.set_option("query_stationary", -1)


def _refsum_cases():
    import glob
    return sorted(glob.glob(os.path.join(GOLDEN, "refsum_gpu_*.npz")))


@pytest.mark.parametrize("path", _refsum_cases(), ids=lambda p: os.path.basename(p)[11:-4])
def test_join_against_reference_gpu_digest(gpu_join, oracle_mod, path):
    # A full-size run of the reference's own kernels on a B200 (benchmark configuration 2's shape:
    # 100,000 unit vectors x 384), kept as pair count + order-independent digests of the pair list.
    from test_oracle_golden import _golden_dataset, _key_digests
    g = np.load(path)
    pts = _golden_dataset(oracle_mod, g)
    gpu_join.set_points(pts)
    st = gpu_join.join(float(g["epsilon"]))
    got = gpu_join.pairs()
    assert int(st.pairs_found) == int(g["pairs_found"]) == len(got)
    ksum, kxor = _key_digests(got)
    assert ksum == int(g["key_sum"]) and kxor == int(g["key_xor_mix"])
    assert np.array_equal(got[:4096], g["first_pairs"])


@pytest.mark.parametrize("n,d,eps", [(256, 64, 1e3), (300, 100, 1e3), (1000, 256, 0.5), (2000, 512, 0.7),
                                     (4096, 128, 0.3136), (777, 333, 0.5), (3000, 2048, 1.6)])
def test_cta_pair_kernel_is_bit_identical(gpu_join, oracle_mod, n, d, eps):
    # The 2-CTA (cta_group::2) kernel computes the same accumulators in the same K order:
    # pairs and emitted distances must equal the single-CTA kernel's bit for bit.
    rng = np.random.default_rng(n + d)
    pts = oracle_mod.double_to_half(rng.exponential(1 / 40.0, size=(n, d)))
    gpu_join.set_points(pts)
    try:
        gpu_join.set_option("cta_pair", 0)
        a = gpu_join.join(eps, capacity=n * n, flags=1)
        pa, da = gpu_join.pairs(with_dist2=True)
        gpu_join.set_option("cta_pair", 1)
        b = gpu_join.join(eps, capacity=n * n, flags=1)
        pb, db = gpu_join.pairs(with_dist2=True)
        # bands too
        gpu_join.join(eps, q_begin=128, q_end=min(n, 600), capacity=n * n)
        band = gpu_join.pairs()
    finally:
        gpu_join.set_option("cta_pair", 0)
    assert a.status == b.status == 0 and a.pairs_found == b.pairs_found
    assert np.array_equal(pa, pb) and np.array_equal(da.view(np.uint32), db.view(np.uint32))
    assert np.array_equal(band, pa[(pa[:, 0] >= 128) & (pa[:, 0] < min(n, 600))])


@pytest.mark.parametrize("n,d,eps", [(256, 64, 1e3), (300, 100, 1e3), (1000, 256, 0.5), (4096, 128, 0.3136),
                                     (777, 333, 0.5), (5000, 1024, 1.1), (9000, 64, 0.2)])
def test_symmetric_schedule_is_bit_identical(gpu_join, oracle_mod, n, d, eps):
    # Computing each unordered pair once and emitting both orientations must give exactly the
    # full join's output: same pairs, same FP32 distances (d2(i,j) and d2(j,i) agree bit for bit).
    from fasted_b200 import FastedError
    rng = np.random.default_rng(3 * n + d)
    pts = oracle_mod.double_to_half(rng.exponential(1 / 40.0, size=(n, d)))
    gpu_join.set_points(pts)
    a = gpu_join.join(eps, capacity=n * n, flags=1)
    pa, da = gpu_join.pairs(with_dist2=True)
    b = gpu_join.join(eps, capacity=n * n, flags=1 | 8)
    pb, db = gpu_join.pairs(with_dist2=True)
    assert a.pairs_found == b.pairs_found and b.status == 0
    assert np.array_equal(pa, pb) and np.array_equal(da.view(np.uint32), db.view(np.uint32))
    with pytest.raises(FastedError):
        gpu_join.join(eps, q_begin=0, q_end=n - 1, flags=8)  # only defined for the full self-join


def test_fp64_brute_force_pairs_match_cpu_truth(gpu_join, oracle_mod):
    pts = oracle_mod.gen_exponential(3000, 128)
    gpu_join.set_points(pts)
    rows = np.arange(1000, 1064, dtype=np.int32)
    counts, pairs = gpu_join.brute_force_pairs(rows, 0.3, capacity=64 * 3000)
    want, _, _ = oracle_mod.join_fp64(pts, 0.3, q_begin=1000, q_end=1064)
    cmp = oracle_mod.compare_pair_sets(pts, 128, 0.3, pairs, want, band=1e-9)
    assert cmp["ok"] and int(counts.sum()) == len(pairs)


def test_estimate_epsilon_hits_target(gpu_join, oracle_mod):
    gpu_join.generate_exponential(30_000, 256)
    eps, got = gpu_join.estimate_epsilon(24.0, sample_rows=4096, rel_tol=0.02)
    assert abs(got - 24.0) <= 0.02 * 24.0 + 1e-9
    st = gpu_join.join(eps, flags=2)
    full_mean = (st.pairs_found - 30_000) / 30_000
    assert 0.8 * 24 <= full_mean <= 1.25 * 24  # the sample (8 bands) speaks for the whole set
    from fasted_b200 import FastedError
    with pytest.raises(FastedError):
        gpu_join.estimate_epsilon(0.0)


def test_full_size_headline_shape_properties(gpu_join, oracle_mod):
    # The benchmark's own shape (1,000,000 x 4096, ~57 M pairs): too large for any CPU oracle, so
    # size-independent properties: row-major order, symmetry, the diagonal, no padding index, and
    # sampled query rows against the FP64 brute force on the device (band rule for disagreements).
    n, d = 1_000_000, 4096
    gpu_join.generate_exponential(n, d)
    eps = 2.1143826828408416  # ~56 neighbours per point on this seeded dataset
    st = gpu_join.join(eps, flags=8)  # symmetric schedule: bit-identical output, half the time
    assert st.status == 0 and st.pairs_found == st.pairs_stored
    assert 40 * n < st.pairs_found < 80 * n
    got = gpu_join.pairs()
    keys = (got[:, 0].astype(np.int64) << 32) | got[:, 1].astype(np.int64)
    assert (np.diff(keys) > 0).all()
    assert got.min() >= 0 and got.max() < n
    assert int((got[:, 0] == got[:, 1]).sum()) == n
    # symmetry: every off-diagonal pair appears in both orientations
    up = got[got[:, 0] < got[:, 1]]
    lo = got[got[:, 0] > got[:, 1]]
    assert len(up) == len(lo)
    ku = (up[:, 0].astype(np.int64) << 32) | up[:, 1].astype(np.int64)
    kl = np.sort((lo[:, 1].astype(np.int64) << 32) | lo[:, 0].astype(np.int64))
    assert np.array_equal(ku, kl)
    del keys, up, lo, ku, kl
    # sampled rows vs FP64 truth: every disagreement must sit inside the 1e-3 band around eps^2
    # (the bit-exact check of this shape against the oracle is test_full_size_band_is_bit_identical_to_the_oracle)
    rows = np.arange(123_456, 123_456 + 48, dtype=np.int32)
    counts, truth = gpu_join.brute_force_pairs(rows, eps, capacity=48 * 65536)
    mine = got[(got[:, 0] >= rows[0]) & (got[:, 0] <= rows[-1])]
    kt = (truth[:, 0].astype(np.int64) << 32) | truth[:, 1].astype(np.int64)
    km = (mine[:, 0].astype(np.int64) << 32) | mine[:, 1].astype(np.int64)
    only = np.concatenate([np.setdiff1d(kt, km), np.setdiff1d(km, kt)])
    if len(only):
        pr = np.stack([only >> 32, only & 0xFFFFFFFF], 1)
        sub = gpu_join.get_rows(np.unique(pr.ravel()))
        lut = {int(r): i for i, r in enumerate(np.unique(pr.ravel()))}
        f = sub.view(np.float16).astype(np.float64)
        d2 = np.array([((f[lut[int(a)]] - f[lut[int(b)]]) ** 2).sum() for a, b in pr])
        assert (np.abs(d2 - eps * eps) <= BAND * eps * eps).all()


def _free_host_bytes():
    import psutil
    return psutil.virtual_memory().available


@pytest.mark.parametrize("name,q_begin,rows", [("c2", 40_960, 256), ("c3", 500_096, 64), ("c4", 1_200_000 // 128 * 128, 64),
                                               ("c5", 2_345_600, 64)])
def test_full_size_band_is_bit_identical_to_the_oracle(gpu_join, oracle_mod, name, q_begin, rows):
    # The benchmark's own configurations at FULL size (the same seeded data bench.py generates): a band
    # of query rows against all N candidates must give exactly the oracle's pairs AND its FP32 squared
    # distances, bit for bit.  The whole matrix is copied to the host once; the oracle evaluates the
    # accumulate model wherever a conservative screen cannot rule a pair out (oracle.join_band_screened,
    # pinned against the plain restatement by the CPU tests).
    import torch
    from fasted_b200.workloads import WORKLOADS, fill_device, padded_dim
    wl = WORKLOADS[name]
    n, d = wl["n"], wl["d"]
    ld = padded_dim(d)
    need_dev = n * ld * 2 + rows * wl.get("pairs_per_point", 256) * 64
    need_host = n * d * 2 * 2 + (4 << 30)
    if torch.cuda.mem_get_info()[0] < need_dev + (8 << 30) or _free_host_bytes() < need_host:
        pytest.skip("not enough free device or host memory for this configuration")
    dev = torch.zeros((n, ld), dtype=torch.float16, device="cuda")
    fill_device(gpu_join, dev, wl)
    torch.cuda.synchronize()
    gpu_join.set_points_device(dev.data_ptr(), n, d, ld, keepalive=dev)
    try:
        eps = wl["eps"]
        if eps is None:
            eps, _ = gpu_join.estimate_epsilon(wl["target"], 4096, 0.02)
        cap = rows * max(8192, 4 * wl.get("pairs_per_point", 256))
        st = gpu_join.join(eps, q_begin=q_begin, q_end=q_begin + rows, capacity=cap, flags=1)
        assert st.status == 0 and st.pairs_found == st.pairs_stored >= rows
        got, got_d2 = gpu_join.pairs(with_dist2=True)
        # the streaming entry point on the same band: identical list
        sgot = np.full((len(got), 2), -1, dtype=np.int32)
        gpu_join.join_stream(eps, q_begin=q_begin, q_end=q_begin + rows, capacity=cap, pairs_host=sgot.ctypes.data,
                             host_capacity=len(got))
        assert np.array_equal(sgot, got)
        host = np.empty((n, d), dtype=np.uint16)
        gpu_join.get_points_into(host.ctypes.data, d)
        norms_gpu, _ = gpu_join.row_norms()
    finally:
        gpu_join.set_points(np.zeros((1, 64), dtype=np.uint16))  # drop the borrowed matrix
        del dev
        torch.cuda.empty_cache()
    norms = oracle_mod.row_norms(host, d)
    assert np.array_equal(norms_gpu.view(np.uint32), norms.view(np.uint32))  # all N row norms, bit for bit
    want, want_d2 = oracle_mod.join_band_screened(host, eps, q_begin, q_begin + rows, d=d, norms=norms)
    assert len(want) >= rows * min(wl["target"], 4) // 4 + rows  # the band has real neighbours, not only self pairs
    assert np.array_equal(got, want), (len(got), len(want))
    assert np.array_equal(got_d2.view(np.uint32), want_d2.view(np.uint32))


@pytest.mark.parametrize("n,d,eps,world", [(5000, 128, 0.33, 2), (9000, 64, 0.2, 3), (20000, 256, 0.45, 8)])
def test_symmetric_shards_union_is_the_full_join(gpu_join, oracle_mod, n, d, eps, world):
    # The multi-GPU symmetric schedule, shard by shard on one GPU: the shards' outputs are disjoint
    # and their union is the full join's output.
    gpu_join.set_points(oracle_mod.gen_exponential(n, d))
    gpu_join.set_option("band_tiles", 2)  # several raster bands even at this size
    try:
        gpu_join.join(eps, capacity=n * 4096)
        want = oracle_mod.pair_keys(gpu_join.pairs())
        parts = []
        for r in range(world):
            st = gpu_join.join_symmetric_shard(eps, r, world, capacity=n * 4096)
            p = gpu_join.pairs()
            assert st.pairs_found == len(p)
            k = oracle_mod.pair_keys(p)
            assert (np.diff(k.astype(np.int64)) > 0).all()
            parts.append(k)
    finally:
        gpu_join.set_option("band_tiles", 0)
    allk = np.concatenate(parts)
    assert len(np.unique(allk)) == len(allk) == len(want)
    assert np.array_equal(np.sort(allk), want)
    sizes = [len(p) for p in parts]
    assert min(sizes) > 0


def test_join_tiny_shapes(gpu_join, oracle_mod):
    # one point, one dimension, duplicates: the smallest inputs the interface accepts
    one = oracle_mod.double_to_half(np.array([[0.25]]))
    gpu_join.set_points(one)
    st = gpu_join.join(0.0)
    assert st.pairs_found == 1 and gpu_join.pairs().tolist() == [[0, 0]]
    two = oracle_mod.double_to_half(np.array([[0.5, 0.125, 0.0], [0.5, 0.125, 0.0]]))
    gpu_join.set_points(two)
    assert gpu_join.join(0.0).pairs_found == 4
    assert gpu_join.pairs().tolist() == [[0, 0], [0, 1], [1, 0], [1, 1]]
    line = oracle_mod.double_to_half(np.arange(300, dtype=np.float64).reshape(300, 1) / 64.0)
    gpu_join.set_points(line)
    gpu_join.join(1.0 / 64.0 + 1e-9)
    got = gpu_join.pairs()
    want, _ = oracle_mod.join_fp16_fp32(line, 1.0 / 64.0 + 1e-9)
    assert np.array_equal(got, want) and len(got) == 300 + 2 * 299
    for flags in (8,):  # the symmetric schedule on the same tiny inputs
        gpu_join.join(1.0 / 64.0 + 1e-9, flags=flags)
        assert np.array_equal(gpu_join.pairs(), want)


@pytest.mark.parametrize("kind,n,d", [("exp", 192, 512), ("exp", 96, 4096), ("gauss", 192, 512), ("wide", 160, 256),
                                      ("unit", 160, 384), ("tiny", 130, 128), ("exp", 200, 100)])
def test_raw_accumulators_match_the_accumulate_model(gpu_join, oracle_mod, kind, n, d):
    # FASTED_JOIN_RAW_DOT returns the FP32 Gram entries as the tensor core left them.  They must equal,
    # bit for bit, the oracle's model of one K=16 instruction: operands aligned to the largest exponent,
    # every term truncated to 26 bits below it, exact sum, truncation to FP32.
    rng = np.random.default_rng(n * d)
    x = {"exp": lambda: rng.exponential(1 / 40.0, size=(n, d)),
         "gauss": lambda: rng.standard_normal((n, d)),
         "wide": lambda: rng.standard_normal((n, d)) * 10.0 ** rng.integers(-3, 3, size=(n, d)),
         "unit": lambda: (lambda v: v / np.linalg.norm(v, axis=1, keepdims=True))(rng.standard_normal((n, d))),
         "tiny": lambda: rng.standard_normal((n, d)) * 1e-5}[kind]()
    pts = oracle_mod.double_to_half(x)
    gpu_join.set_points(pts)
    st = gpu_join.join(1e18, capacity=n * n, flags=1 | 16)
    pairs, a = gpu_join.pairs(with_dist2=True)
    assert st.pairs_found == n * n
    got = np.empty((n, n), dtype=np.float32)
    got[pairs[:, 0], pairs[:, 1]] = a
    want = oracle_mod.gram_matrix(pts)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_accumulate_rule_known_answers(gpu_join, oracle_mod):
    # Crafted K=16 dot products that pin the rule down (each line: what it shows).
    u = 2.0 ** -23  # one FP32 ulp at 1.0

    def vec(pairs, k=16):
        x, y = np.zeros(k), np.zeros(k)
        for i, (a, b) in enumerate(pairs):
            x[i], y[i] = a, b
        return x, y

    cases = [
        # 15 products of half an ulp next to 1.0 are kept (window reaches 2 bits below the ulp): 7.5 -> 7 ulps
        (vec([(1.0, 1.0)] + [(2.0 ** -12, 2.0 ** -12)] * 15), 1 + 7 * u),
        # quarter-ulp products are kept too: 3.75 -> 3 ulps ...
        (vec([(1.0, 1.0)] + [(2.0 ** -12, 2.0 ** -13)] * 15), 1 + 3 * u),
        # ... eighth-ulp products fall out of the window one by one: 1.875 ulps vanish
        (vec([(1.0, 1.0)] + [(2.0 ** -13, 2.0 ** -13)] * 15), 1.0),
        # the window hangs on the exponent SUM of the operands: 1.5 * 1.5 = 2.25 still keeps 2^-25 terms
        (vec([(1.5, 1.5)] + [(2.0 ** -12, 2.0 ** -13)] * 8), 2.25 + 8 * 2.0 ** -25),
        # 1.5 * 2 = 3 has exponent sum 1: 2^-25 terms vanish, 2^-24 terms stay
        (vec([(1.5, 2.0)] + [(2.0 ** -12, 2.0 ** -13)] * 8), 3.0),
        (vec([(1.5, 2.0)] + [(2.0 ** -12, 2.0 ** -12)] * 8), 3.0 + 8 * 2.0 ** -24),
        # each term is truncated toward zero (a small negative term is dropped, not rounded down) ...
        (vec([(1.0, 1.0), (-2.0 ** -13, 2.0 ** -13)]), 1.0),
        # ... partial terms lose their low bits: 8 x 1.5 * 2^-25 counts as 8 x 2^-25
        (vec([(1.0, 1.0)] + [(1.5 * 2.0 ** -12, 2.0 ** -13)] * 8), 1 + 2 * u),
        # the final sum is truncated toward zero as well, for both signs
        (vec([(1.0, 1.0), (2.0 ** -11, 0.75 * 2.0 ** -12)]), 1.0),
        (vec([(-1.0, 1.0), (-2.0 ** -11, 1.75 * 2.0 ** -12)]), -(1 + u)),
        # the accumulator of the previous instruction is one more aligned term (K = 32):
        # 1.0 first, then sixteen 2^-26 terms: all dropped; the other way round they add up exactly first
        (vec([(1.0, 1.0)] + [(0, 0)] * 15 + [(2.0 ** -13, 2.0 ** -13)] * 16, 32), 1.0),
        (vec([(2.0 ** -13, 2.0 ** -13)] * 16 + [(0, 0)] * 15 + [(1.0, 1.0)], 32), 1 + 2 * u),
    ]
    for (x, y), want in cases:
        pts = oracle_mod.double_to_half(np.stack([x, y]))
        assert np.array_equal(oracle_mod.half_to_float(pts).astype(np.float64), np.stack([x, y]))
        gpu_join.set_points(pts)
        gpu_join.join(1e18, capacity=4, flags=1 | 16)
        pairs, a = gpu_join.pairs(with_dist2=True)
        got = float(a[(pairs[:, 0] == 0) & (pairs[:, 1] == 1)][0])
        assert got == want, (x[:4], y[:4], got, want)
        assert float(oracle_mod.gram_matrix(pts)[0, 1]) == want
