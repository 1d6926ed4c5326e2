"""The join epilogue first applies a cheap conservative test and runs the exact distance test only
where that one does not reject.  This checks the bound on the host in emulated FP32: whenever the
exact expression d2 = RN(RN(sq + sc) - 2a) is <= eps2, the cheap expression
RN(RN(sc - 2a) + sq) must NOT exceed eps2 + 2^-19 * (sq + max_sc + eps2).  Values are drawn so that
d2 lands within a few ulps of eps2, where the two roundings differ most."""
import numpy as np

SLACK = np.float32(2.0 ** -19)  # kRejectSlack in fasted_b200/csrc/kernels.cuh


def _f32(x):
    return np.asarray(x, dtype=np.float64).astype(np.float32)


def _check(sq, sc, a, eps2, max_sc=None):
    sq, sc, a = _f32(sq), _f32(sc), _f32(a)
    eps2 = np.float32(eps2)
    t = (sq + sc).astype(np.float32)                                   # RN(sq + sc)
    d2 = _f32(t.astype(np.float64) - 2.0 * a.astype(np.float64))        # one rounding: fma(a, -2, t)
    u = _f32(sc.astype(np.float64) - 2.0 * a.astype(np.float64))        # fma(a, -2, sc)
    fast = (u + sq).astype(np.float32)
    mx = sc if max_sc is None else np.maximum(sc, np.float32(max_sc))
    thr = _f32(SLACK.astype(np.float64) * ((sq + (mx + eps2).astype(np.float32)).astype(np.float32)).astype(np.float64)
               + np.float64(eps2))
    hit = d2 <= eps2
    rejected = fast > thr
    bad = hit & rejected
    assert not bad.any(), (sq[bad][:3], sc[bad][:3], a[bad][:3], eps2)
    return int(hit.sum()), int((~rejected).sum())


def test_no_hit_is_rejected_near_the_threshold():
    rng = np.random.default_rng(7)
    hits = passed = 0
    for scale in [1e-6, 1e-3, 0.3, 5.0, 300.0, 6e4]:
        for eps_rel in [1e-4, 0.05, 0.9, 3.0]:
            n = 400_000
            sq = rng.uniform(0.5, 1.5, n) * scale
            sc = rng.uniform(0.5, 1.5, n) * scale
            eps2 = np.float32(scale * eps_rel)
            # a such that the real sq + sc - 2a sits within +-8 ulps of eps2
            ulp = np.spacing(np.float32(max(scale * 3, float(eps2))))
            delta = rng.integers(-8, 9, n) * ulp * rng.uniform(0, 1, n)
            a = (sq + sc - (eps2 + delta)) / 2.0
            h, p = _check(sq, sc, a, eps2, max_sc=1.5 * scale)
            hits += h
            passed += p
    assert hits > 1_000_000 and passed >= hits


def test_extremes_do_not_reject_hits():
    rng = np.random.default_rng(11)
    n = 200_000
    # zero vectors, huge dot products (a much larger than the norms), negative dot products
    z = np.zeros(n)
    _check(z, z, z, 1e-6)
    sq = rng.uniform(0, 10, n)
    sc = rng.uniform(0, 10, n)
    _check(sq, sc, rng.uniform(50, 1e6, n), 0.5)          # d2 very negative: always a hit
    _check(sq, sc, -rng.uniform(0, 1e3, n), 1e30)         # everything within a huge eps
    _check(sq, sc, np.sqrt(sq * sc), 0.0)                 # eps = 0: only exact coincidences
