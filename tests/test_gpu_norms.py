"""Row-norm kernel vs the oracle: bit-exact (FP32 round-toward-zero chain)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,d", [(1, 1), (7, 2), (128, 64), (129, 65), (300, 100), (1000, 64), (513, 384),
                                 (2048, 128), (257, 1000), (4096, 128), (100, 4096), (3000, 777)])
def test_norms_bit_exact(gpu_join, oracle_mod, n, d):
    rng = np.random.default_rng(n * 7919 + d)
    vals = rng.exponential(1 / 40.0, size=(n, d))
    if d > 2:
        vals[:, 1] *= -1  # signs must not matter
    pts = oracle_mod.double_to_half(vals)
    gpu_join.set_points(pts)
    got, ms = gpu_join.row_norms()
    want = oracle_mod.row_norms(pts)
    assert got.dtype == np.float32 and got.shape == (n,)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert ms >= 0


def test_norms_increasing_integers_known_answer(gpu_join, oracle_mod):
    # tests/python/sumSquared/sumSquared.py:3-11 of the reference (matrix of source/main.cu:86-104)
    vals = np.arange(32 * 64, dtype=np.float64).reshape(32, 64)
    pts = oracle_mod.double_to_half(vals)
    gpu_join.set_points(pts)
    got, _ = gpu_join.row_norms()
    want = (vals ** 2).sum(axis=1)
    exact = want < 2 ** 24
    assert np.array_equal(got[exact].astype(np.float64), want[exact])
    assert np.array_equal(got, oracle_mod.row_norms(pts))


def test_norms_reference_dataset(gpu_join, oracle_mod):
    pts = oracle_mod.gen_exponential(4096, 128)
    gpu_join.set_points(pts)
    got, _ = gpu_join.row_norms()
    assert np.array_equal(got, oracle_mod.row_norms(pts))


def test_norms_large_property(gpu_join):
    # Size-independent property at a larger size: device-generated data, norms of duplicated
    # halves are equal and every norm is within RZ bounds of the FP64 sum.
    gpu_join.generate_exponential(200_000, 512)
    pts = gpu_join.get_points()
    got, ms = gpu_join.row_norms()
    f = pts.view(np.float16).astype(np.float64)
    want = (f * f).sum(axis=1)
    rel = (want - got) / want
    assert (rel > -1e-7).all() and (rel < 512 * 2.0 ** -23).all()


def test_exact_norms_option_is_correctly_rounded(gpu_join, oracle_mod):
    # Opt-in mode (not the reference's numerics): FP64 sum of the exact squares, one rounding.
    rng = np.random.default_rng(9)
    pts = oracle_mod.double_to_half(rng.exponential(1 / 40.0, size=(700, 1000)))
    gpu_join.set_points(pts)
    try:
        gpu_join.set_option("exact_norms", 1)
        got, _ = gpu_join.row_norms()
    finally:
        gpu_join.set_option("exact_norms", 0)
    f = pts.view(np.float16).astype(np.float64)
    want = (f * f).sum(axis=1).astype(np.float32)
    assert np.array_equal(got, want)
    ref, _ = gpu_join.row_norms()
    assert np.array_equal(ref, oracle_mod.row_norms(pts)) and (ref <= got).all() and (ref < got).any()


def test_large_pageable_upload_and_download_round_trip(gpu_join, oracle_mod):
    # Above 8 MB, pageable host memory travels through the pinned staging buffers (both pitches).
    rng = np.random.default_rng(4)
    big = rng.integers(0, 0x7BFF, size=(150_000, 200), dtype=np.uint16)  # 60 MB, d not a multiple of 64
    gpu_join.set_points(big)
    assert np.array_equal(gpu_join.get_points(), big)
    wide = np.zeros((90_000, 320), dtype=np.uint16)
    wide[:, :300] = rng.integers(0, 0x7BFF, size=(90_000, 300), dtype=np.uint16)
    gpu_join.set_points(wide, d=300)  # row stride 320 on the host, 300 real columns
    assert np.array_equal(gpu_join.get_points(), wide[:, :300])
    norms, _ = gpu_join.row_norms()
    assert np.array_equal(norms[:2000], oracle_mod.row_norms(np.ascontiguousarray(wide[:2000, :300])))
