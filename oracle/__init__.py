"""CPU oracle for the epsilon self-join -- TEST INFRASTRUCTURE ONLY.

ctypes front end of ``oracle/liboracle.so`` (built from ``oracle/oracle.cpp`` by
``make -C oracle``).  It restates the reference's FP16 -> FP32 join on the CPU
and provides the FP64 brute-force join used as ground truth and timed CPU
baseline.  Only the tests, the smoke check and the benchmark's ``cpu_baseline``
/ ``--impl reference`` legs may import this module; the product package never
does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

_i64 = ctypes.c_int64
_u64 = ctypes.c_uint64
_vp = ctypes.c_void_p


def build(force: bool = False) -> str:
    """Compile liboracle.so (g++, OpenMP) if missing or stale."""
    src = os.path.join(_HERE, "oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        L.oracle_gen_exponential.argtypes = [_i64, _i64, ctypes.c_double, ctypes.c_double, _vp, _i64]
        L.oracle_gen_exponential.restype = None
        L.oracle_double_to_half.argtypes = [_vp, _i64, _vp]
        L.oracle_half_to_float.argtypes = [_vp, _i64, _vp]
        L.oracle_read_csv.argtypes = [ctypes.c_char_p, ctypes.POINTER(_i64), ctypes.POINTER(_i64), _vp, _i64]
        L.oracle_read_csv.restype = ctypes.c_int
        L.oracle_fnv1a64_u16.argtypes = [_vp, _i64, _u64]
        L.oracle_fnv1a64_u16.restype = _u64
        L.oracle_row_norms.argtypes = [_vp, _i64, _i64, _i64, _vp]
        L.oracle_join_fp16_fp32.argtypes = [_vp, _i64, _i64, _i64, _vp, ctypes.c_double, _i64, _i64, _vp, _vp, _u64]
        L.oracle_join_fp16_fp32.restype = _u64
        L.oracle_join_band_screened.argtypes = [_vp, _i64, _i64, _i64, _vp, ctypes.c_double, _i64, _i64, _vp, _vp, _u64]
        L.oracle_join_band_screened.restype = _u64
        L.oracle_join_fp64.argtypes = [_vp, _i64, _i64, _i64, ctypes.c_double, _i64, _i64, _vp, _vp, _u64]
        L.oracle_join_fp64.restype = _u64
        L.oracle_gram_matrix.argtypes = [_vp, _i64, _i64, _i64, _i64, _i64, _vp]
        L.oracle_gram_matrix.restype = None
        L.oracle_pair_d2_fp64.argtypes = [_vp, _i64, _i64, _vp, _i64, _vp]
        L.oracle_num_threads.restype = ctypes.c_int
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(_vp)


def _check_pts(pts: np.ndarray) -> np.ndarray:
    assert pts.dtype == np.uint16 and pts.ndim == 2 and pts.flags.c_contiguous
    return pts


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def gen_exponential(n: int, d: int, lam: float = 40.0, max_value: float = 10.0, ld: int | None = None) -> np.ndarray:
    """The reference's seeded ``-e`` dataset as binary16 bit patterns, shape (n, ld)."""
    ld = d if ld is None else ld
    out = np.empty((n, ld), dtype=np.uint16)
    lib().oracle_gen_exponential(n, d, lam, max_value, _p(out), ld)
    return out


def double_to_half(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float64)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_double_to_half(_p(x), x.size, _p(out))
    return out


def half_to_float(h: np.ndarray) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, dtype=np.float32)
    lib().oracle_half_to_float(_p(h), h.size, _p(out))
    return out


def read_csv(path: str, dim_multiple: int = 1) -> tuple[np.ndarray, int]:
    """CSV -> (binary16 bits of shape (n, ld), d) with ld = d rounded up to dim_multiple."""
    n, d = _i64(0), _i64(0)
    rc = lib().oracle_read_csv(path.encode(), ctypes.byref(n), ctypes.byref(d), None, 0)
    if rc:
        raise RuntimeError(f"oracle_read_csv failed with code {rc}")
    ld = -(-d.value // dim_multiple) * dim_multiple
    out = np.zeros((n.value, ld), dtype=np.uint16)
    rc = lib().oracle_read_csv(path.encode(), ctypes.byref(n), ctypes.byref(d), _p(out), ld)
    if rc:
        raise RuntimeError(f"oracle_read_csv failed with code {rc}")
    return out, d.value


def fnv1a64_u16(h: np.ndarray, seed: int = 0) -> int:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    return int(lib().oracle_fnv1a64_u16(_p(h), h.size, seed))


def row_norms(pts: np.ndarray, d: int | None = None) -> np.ndarray:
    """Reference row norms (sequential round-toward-zero FP32), shape (n,)."""
    _check_pts(pts)
    n, ld = pts.shape
    d = ld if d is None else d
    out = np.empty(n, dtype=np.float32)
    lib().oracle_row_norms(_p(pts), n, d, ld, _p(out))
    return out


def gram_matrix(pts: np.ndarray, d: int | None = None, r_begin: int = 0, r_end: int | None = None) -> np.ndarray:
    """Raw FP32 Gram entries under the measured tensor-core accumulate model, rows [r_begin, r_end) x all."""
    _check_pts(pts)
    n, ld = pts.shape
    d = ld if d is None else d
    r_end = n if r_end is None else r_end
    out = np.empty((r_end - r_begin, n), dtype=np.float32)
    lib().oracle_gram_matrix(_p(pts), n, d, ld, r_begin, r_end, _p(out))
    return out


def join_fp16_fp32(pts: np.ndarray, eps: float, d: int | None = None, q_begin: int = 0, q_end: int | None = None,
                   norms: np.ndarray | None = None):
    """Reference algorithm restated on the CPU.  Returns (pairs[int32 (m,2)], d2[float32 (m,)]) row-major."""
    _check_pts(pts)
    n, ld = pts.shape
    d = ld if d is None else d
    q_end = n if q_end is None else q_end
    if norms is None:
        norms = row_norms(pts, d)
    norms = np.ascontiguousarray(norms, dtype=np.float32)
    found = lib().oracle_join_fp16_fp32(_p(pts), n, d, ld, _p(norms), eps, q_begin, q_end, None, None, 0)
    pairs = np.empty((found, 2), dtype=np.int32)
    d2 = np.empty(found, dtype=np.float32)
    lib().oracle_join_fp16_fp32(_p(pts), n, d, ld, _p(norms), eps, q_begin, q_end, _p(pairs), _p(d2), found)
    return pairs, d2


def join_band_screened(pts: np.ndarray, eps: float, q_begin: int, q_end: int, d: int | None = None,
                       norms: np.ndarray | None = None):
    """join_fp16_fp32 for a band of query rows of a large dataset: the same output, with the accumulate
    model evaluated only for entries that a conservative FP32 screen cannot rule out."""
    _check_pts(pts)
    n, ld = pts.shape
    d = ld if d is None else d
    if norms is None:
        norms = row_norms(pts, d)
    norms = np.ascontiguousarray(norms, dtype=np.float32)
    found = lib().oracle_join_band_screened(_p(pts), n, d, ld, _p(norms), eps, q_begin, q_end, None, None, 0)
    pairs = np.empty((found, 2), dtype=np.int32)
    d2 = np.empty(found, dtype=np.float32)
    lib().oracle_join_band_screened(_p(pts), n, d, ld, _p(norms), eps, q_begin, q_end, _p(pairs), _p(d2), found)
    return pairs, d2


def join_fp64(pts: np.ndarray, eps: float, d: int | None = None, q_begin: int = 0, q_end: int | None = None,
              capacity: int | None = None):
    """FP64 brute force.  Returns (pairs[int32 (m,2)], d2[float64 (m,)], found)."""
    _check_pts(pts)
    n, ld = pts.shape
    d = ld if d is None else d
    q_end = n if q_end is None else q_end
    if capacity is None:
        capacity = int(lib().oracle_join_fp64(_p(pts), n, d, ld, eps, q_begin, q_end, None, None, 0))
    pairs = np.empty((capacity, 2), dtype=np.int32)
    d2 = np.empty(capacity, dtype=np.float64)
    found = int(lib().oracle_join_fp64(_p(pts), n, d, ld, eps, q_begin, q_end, _p(pairs), _p(d2), capacity))
    m = min(found, capacity)
    return pairs[:m], d2[:m], found


def pair_d2_fp64(pts: np.ndarray, pairs: np.ndarray, d: int | None = None) -> np.ndarray:
    _check_pts(pts)
    n, ld = pts.shape
    d = ld if d is None else d
    pairs = np.ascontiguousarray(pairs, dtype=np.int32).reshape(-1, 2)
    out = np.empty(len(pairs), dtype=np.float64)
    lib().oracle_pair_d2_fp64(_p(pts), d, ld, _p(pairs), len(pairs), _p(out))
    return out


def pair_keys(pairs: np.ndarray) -> np.ndarray:
    """(q, c) int32 pairs -> uint64 keys q << 32 | c (row-major order == numeric order)."""
    p = np.ascontiguousarray(pairs, dtype=np.int64).reshape(-1, 2)
    return (p[:, 0].astype(np.uint64) << np.uint64(32)) | p[:, 1].astype(np.uint64)


def compare_pair_sets(pts: np.ndarray, d: int, eps: float, pairs_a: np.ndarray, pairs_b: np.ndarray,
                      band: float = 1e-3) -> dict:
    """Set difference of two pair lists, with every disagreement checked against the band.

    A pair present in only one list is *excused* when its FP64 squared distance lies within
    ``band * eps^2`` of ``eps^2``.  Returns counts and the unexcused pairs.
    """
    ka, kb = pair_keys(pairs_a), pair_keys(pairs_b)
    only_a = np.setdiff1d(ka, kb, assume_unique=False)
    only_b = np.setdiff1d(kb, ka, assume_unique=False)
    eps2 = eps * eps

    def unexcused(keys):
        if len(keys) == 0:
            return np.empty((0, 2), dtype=np.int32)
        pr = np.stack([(keys >> np.uint64(32)).astype(np.int32), (keys & np.uint64(0xFFFFFFFF)).astype(np.int32)], 1)
        d2 = pair_d2_fp64(pts, pr, d)
        bad = np.abs(d2 - eps2) > band * eps2
        return pr[bad]

    ua, ub = unexcused(only_a), unexcused(only_b)
    return {
        "n_a": int(len(ka)), "n_b": int(len(kb)),
        "only_a": int(len(only_a)), "only_b": int(len(only_b)),
        "unexcused_a": ua, "unexcused_b": ub,
        "ok": len(ua) == 0 and len(ub) == 0,
    }
