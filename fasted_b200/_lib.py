"""ctypes binding of the native library's context API (include/fasted.h, layer 2).

The library is CUDA-only: loading works anywhere (so that symbol checks can run
on a machine without a GPU), every compute call fails loudly without an sm_100
device.  There is no CPU fallback in this package.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libfasted.so")
LEGACY_LIB_PATH = os.path.join(_HERE, "lib", "main.so")

_i64 = ctypes.c_int64
_u64 = ctypes.c_uint64
_vp = ctypes.c_void_p

OK, EINVAL, ECUDA, ENODEV, ESTATE, EKERNEL, EIO = 0, -1, -2, -3, -4, -5, -6
JOIN_DIST2, JOIN_NO_SORT, JOIN_KEEP_NORMS, JOIN_SYMMETRIC = 1, 2, 4, 8


class FastedError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"fasted error {code}: {message}")
        self.code = code


class JoinStats(ctypes.Structure):
    _fields_ = [
        ("pairs_found", ctypes.c_ulonglong),
        ("pairs_stored", ctypes.c_ulonglong),
        ("norms_ms", ctypes.c_double),
        ("join_ms", ctypes.c_double),
        ("kernel_ms", ctypes.c_double),
        ("sort_ms", ctypes.c_double),
        ("status", ctypes.c_ulonglong),
        ("tiles_m", ctypes.c_int),
        ("tiles_n", ctypes.c_int),
        ("grid", ctypes.c_int),
        ("cta0_cycles", ctypes.c_ulonglong),
        ("cta0_tiles", ctypes.c_ulonglong),
        ("cta0_setup_cycles", ctypes.c_ulonglong),
        ("cta0_release_cycles", ctypes.c_ulonglong),
        ("cta0_feed_wait_cycles", ctypes.c_ulonglong),
        ("cta0_acc_wait_cycles", ctypes.c_ulonglong),
        ("chunks", ctypes.c_int),
        ("tail_ms", ctypes.c_double),
    ]

    def as_dict(self) -> dict:
        return {k: getattr(self, k) for k, _ in self._fields_}


# Every symbol include/fasted.h declares, layer 1 and layer 2.
DECLARED_SYMBOLS = [
    "runFromExponentialDataset", "runFromFile", "reRun", "releaseResources",
    "fasted_last_error", "fasted_create", "fasted_destroy", "fasted_set_stream",
    "fasted_set_points_host_f16", "fasted_set_points_device_f16", "fasted_generate_exponential",
    "fasted_fill_exponential_device", "fasted_copy_points_from",
    "fasted_points_info", "fasted_get_points_host_f16", "fasted_get_rows_host_f16", "fasted_row_norms", "fasted_get_norms",
    "fasted_join", "fasted_selftest_wait_timeout", "fasted_join_symmetric_shard", "fasted_tile_schedule", "fasted_estimate_epsilon", "fasted_get_pairs", "fasted_pairs_device", "fasted_brute_force_f64", "fasted_brute_force_f64_pairs", "fasted_set_option",
    "fasted_dataset_exponential_f16", "fasted_dataset_csv_shape", "fasted_dataset_csv_f16",
    "fasted_join_static_scratch", "fasted_join_stream", "fasted_tile_schedule_stationary",
    "fasted_broadcast_points",
    "fasted_shared_chunks_bytes", "fasted_shared_chunks_init", "fasted_join_stream_shared", "fasted_shared_chunks_totals",
    "fasted_shared_chunks_init_plan", "fasted_shared_chunks_take", "fasted_shared_chunks_publish",
    "fasted_shared_chunks_offset", "fasted_shared_chunks_fail", "fasted_shared_chunks_range",
    "fasted_shared_chunks_init_arriving", "fasted_join_stream_arriving",
]

class Arrival(ctypes.Structure):
    """fasted_arrival of include/fasted.h: how the dataset reaches the GPUs while the join starts."""
    _fields_ = [("pieces", ctypes.c_int), ("groups", ctypes.c_int), ("group_rows", ctypes.c_int64),
                ("own_begin", ctypes.c_int64), ("lead_rows", ctypes.c_int64), ("events", ctypes.POINTER(ctypes.c_void_p))]

    @classmethod
    def make(cls, pieces: int, groups: int, group_rows: int, own_begin: int, lead_rows: int = 0, events=None) -> "Arrival":
        a = cls(pieces, groups, group_rows, own_begin, lead_rows, None)
        if events is not None:
            if len(events) != pieces:
                raise ValueError("one event per piece")
            a._handles = (ctypes.c_void_p * pieces)(*[ctypes.c_void_p(int(e) if e else None) for e in events])
            a.events = ctypes.cast(a._handles, ctypes.POINTER(ctypes.c_void_p))
        return a


CHUNK_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64,
                            ctypes.c_uint64)

_lib = None


def load() -> ctypes.CDLL:
    """Load libfasted.so; raises if it has not been built (python -m fasted_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python -m fasted_b200.build` (nvcc, sm_100a). "
            "This package has no fallback implementation.")
    L = ctypes.CDLL(LIB_PATH)
    L.fasted_last_error.restype = ctypes.c_char_p
    L.fasted_create.argtypes = [ctypes.c_int, ctypes.POINTER(_vp)]
    L.fasted_destroy.argtypes = [_vp]
    L.fasted_destroy.restype = None
    L.fasted_set_stream.argtypes = [_vp, _vp]
    L.fasted_set_points_host_f16.argtypes = [_vp, _vp, _i64, _i64, _i64]
    L.fasted_set_points_device_f16.argtypes = [_vp, _vp, _i64, _i64, _i64]
    L.fasted_generate_exponential.argtypes = [_vp, _i64, _i64, ctypes.c_double, ctypes.c_double, _u64]
    L.fasted_copy_points_from.argtypes = [_vp, _vp]
    L.fasted_broadcast_points.argtypes = [ctypes.POINTER(_vp), ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
    L.fasted_fill_exponential_device.argtypes = [_vp, _vp, _i64, _i64, _i64, ctypes.c_double, ctypes.c_double, _u64]
    L.fasted_points_info.argtypes = [_vp, ctypes.POINTER(_vp), ctypes.POINTER(_i64), ctypes.POINTER(_i64),
                                     ctypes.POINTER(_i64)]
    L.fasted_get_points_host_f16.argtypes = [_vp, _vp, _i64]
    L.fasted_get_rows_host_f16.argtypes = [_vp, _vp, _i64, _vp, _i64]
    L.fasted_row_norms.argtypes = [_vp, ctypes.POINTER(ctypes.c_double)]
    L.fasted_get_norms.argtypes = [_vp, _vp]
    L.fasted_join.argtypes = [_vp, ctypes.c_double, _i64, _i64, _u64, ctypes.c_uint, ctypes.POINTER(JoinStats)]
    L.fasted_join_stream.argtypes = [_vp, ctypes.c_double, _i64, _i64, _u64, ctypes.c_uint, _vp, _vp, _u64, CHUNK_FN,
                                     _vp, ctypes.POINTER(JoinStats)]
    L.fasted_shared_chunks_bytes.argtypes = [_u64]
    L.fasted_shared_chunks_bytes.restype = ctypes.c_size_t
    L.fasted_shared_chunks_init.argtypes = [_vp, _vp, ctypes.c_size_t, ctypes.c_double, _i64, _i64, ctypes.c_int,
                                            ctypes.POINTER(_u64)]
    L.fasted_join_stream_shared.argtypes = [_vp, ctypes.c_double, _u64, ctypes.c_uint, _vp, _vp, _u64,
                                            ctypes.POINTER(JoinStats)]
    L.fasted_shared_chunks_totals.argtypes = [_vp, ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(ctypes.c_ulonglong),
                                              ctypes.POINTER(ctypes.c_ulonglong)]
    L.fasted_shared_chunks_init_plan.argtypes = [_vp, ctypes.c_size_t, _i64, _i64, _i64, _i64, ctypes.c_int,
                                                 ctypes.POINTER(_u64)]
    L.fasted_shared_chunks_range.argtypes = [_vp, _u64, ctypes.POINTER(_i64), ctypes.POINTER(_i64)]
    L.fasted_shared_chunks_init_arriving.argtypes = [_vp, _vp, ctypes.c_size_t, ctypes.c_double, ctypes.c_int,
                                                     ctypes.POINTER(Arrival), ctypes.POINTER(_u64)]
    L.fasted_join_stream_arriving.argtypes = [_vp, ctypes.c_double, _u64, ctypes.c_uint, _vp, ctypes.POINTER(Arrival),
                                              _vp, _u64, ctypes.POINTER(JoinStats)]
    L.fasted_shared_chunks_take.argtypes = [_vp]
    L.fasted_shared_chunks_take.restype = _i64
    L.fasted_shared_chunks_publish.argtypes = [_vp, _u64, _u64, _u64]
    L.fasted_shared_chunks_offset.argtypes = [_vp, _u64, ctypes.c_double, ctypes.POINTER(_u64)]
    L.fasted_shared_chunks_fail.argtypes = [_vp]
    L.fasted_shared_chunks_fail.restype = None
    L.fasted_tile_schedule.argtypes = [_i64, _i64, _i64, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                       ctypes.c_int, ctypes.c_int, ctypes.c_int, _vp, _i64, ctypes.POINTER(_i64)]
    L.fasted_tile_schedule_stationary.argtypes = [_i64, _i64, _i64, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                  _vp, _i64, ctypes.POINTER(_i64)]
    L.fasted_join_symmetric_shard.argtypes = [_vp, ctypes.c_double, ctypes.c_int, ctypes.c_int, _u64, ctypes.c_uint,
                                              ctypes.POINTER(JoinStats)]
    L.fasted_selftest_wait_timeout.argtypes = [_vp, ctypes.c_double, ctypes.POINTER(ctypes.c_ulonglong),
                                               ctypes.POINTER(ctypes.c_double)]
    L.fasted_estimate_epsilon.argtypes = [_vp, ctypes.c_double, _i64, ctypes.c_double, ctypes.POINTER(ctypes.c_double),
                                          ctypes.POINTER(ctypes.c_double)]
    L.fasted_get_pairs.argtypes = [_vp, _u64, _u64, _vp, _vp]
    L.fasted_pairs_device.argtypes = [_vp, ctypes.POINTER(_vp), ctypes.POINTER(_vp)]
    L.fasted_brute_force_f64.argtypes = [_vp, _vp, ctypes.c_int, ctypes.c_double, _vp]
    L.fasted_brute_force_f64_pairs.argtypes = [_vp, _vp, ctypes.c_int, ctypes.c_double, _vp, _vp, _u64,
                                               ctypes.POINTER(ctypes.c_ulonglong)]
    L.fasted_set_option.argtypes = [_vp, ctypes.c_char_p, _i64]
    L.fasted_join_static_scratch.argtypes = [_vp, _i64, _i64, _i64, ctypes.c_double, _vp, _u64, _vp,
                                             ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(ctypes.c_ulonglong)]
    L.fasted_dataset_exponential_f16.argtypes = [_i64, _i64, ctypes.c_double, ctypes.c_double, _vp, _i64]
    L.fasted_dataset_csv_shape.argtypes = [ctypes.c_char_p, ctypes.POINTER(_i64), ctypes.POINTER(_i64)]
    L.fasted_dataset_csv_f16.argtypes = [ctypes.c_char_p, _vp, _i64, _i64, _i64]
    _lib = L
    return L


def _check(rc: int) -> None:
    if rc != OK:
        raise FastedError(rc, load().fasted_last_error().decode(errors="replace"))


def dataset_exponential(n: int, d: int, lam: float = 40.0, max_value: float = 10.0) -> np.ndarray:
    """The reference's seeded synthetic dataset (host generator), binary16 bit patterns of shape (n, d)."""
    out = np.empty((n, d), dtype=np.uint16)
    _check(load().fasted_dataset_exponential_f16(n, d, lam, max_value, out.ctypes.data_as(_vp), d))
    return out


def dataset_csv(path: str) -> np.ndarray:
    """CSV dataset with the reference's parsing rules, binary16 bit patterns of shape (n, d)."""
    n, d = _i64(), _i64()
    _check(load().fasted_dataset_csv_shape(path.encode(), ctypes.byref(n), ctypes.byref(d)))
    out = np.empty((n.value, d.value), dtype=np.uint16)
    _check(load().fasted_dataset_csv_f16(path.encode(), out.ctypes.data_as(_vp), n.value, d.value, d.value))
    return out


def join_static_scratch(points_dev: int, n: int, d: int, ld: int, eps: float, keys_out_dev: int, capacity: int,
                        stream: int = 0) -> tuple[int, int]:
    """fasted_join_static_scratch: join on caller-owned device buffers without allocating anything.
    Returns (pairs_found, pairs_stored); records in keys_out_dev are (query << 32) | candidate, unsorted."""
    found, stored = ctypes.c_ulonglong(), ctypes.c_ulonglong()
    _check(load().fasted_join_static_scratch(_vp(points_dev), n, d, ld, float(eps), _vp(keys_out_dev), capacity,
                                             _vp(stream), ctypes.byref(found), ctypes.byref(stored)))
    return int(found.value), int(stored.value)


def tile_schedule(n: int, q_begin: int, q_end: int, grid: int, cta: int, tile_m: int = 128, band_tiles: int = 16,
                  symmetric: bool = False, shard_rank: int = 0, shard_world: int = 1) -> np.ndarray:
    """The (tile row, tile column) sequence one CTA of the join kernel walks (host evaluation, no GPU)."""
    count = _i64()
    _check(load().fasted_tile_schedule(n, q_begin, q_end, tile_m, band_tiles, int(symmetric), shard_rank, shard_world,
                                       grid, cta, None, 0, ctypes.byref(count)))
    out = np.empty((count.value, 2), dtype=np.int32)
    _check(load().fasted_tile_schedule(n, q_begin, q_end, tile_m, band_tiles, int(symmetric), shard_rank, shard_world,
                                       grid, cta, out.ctypes.data_as(_vp), count.value, ctypes.byref(count)))
    return out


def tile_schedule_stationary(n: int, q_begin: int, q_end: int, grid: int, cta: int, rows_per_band: int,
                             symmetric: bool = False) -> np.ndarray:
    """The (tile row, tile column) sequence one CTA of the query-stationary join kernel walks."""
    count = _i64()
    _check(load().fasted_tile_schedule_stationary(n, q_begin, q_end, rows_per_band, int(symmetric), grid, cta, None, 0,
                                                  ctypes.byref(count)))
    out = np.empty((count.value, 2), dtype=np.int32)
    _check(load().fasted_tile_schedule_stationary(n, q_begin, q_end, rows_per_band, int(symmetric), grid, cta,
                                                  out.ctypes.data_as(_vp), count.value, ctypes.byref(count)))
    return out


def broadcast_points(contexts: list["SelfJoin"]) -> float:
    """fasted_broadcast_points: replicate contexts[0]'s dataset into the other contexts (one GPU each, same
    process) with one NCCL broadcast; returns the collective's wall time in milliseconds."""
    arr = (_vp * len(contexts))(*[c._h for c in contexts])
    ms = ctypes.c_double()
    _check(load().fasted_broadcast_points(arr, len(contexts), ctypes.byref(ms)))
    return ms.value


class SelfJoin:
    """One context = one GPU, one resident dataset, repeated joins (the reference's run / reRun cycle)."""

    def __init__(self, device: int = 0):
        self._L = load()
        h = _vp()
        _check(self._L.fasted_create(device, ctypes.byref(h)))
        self._h = h
        self.device = device
        self._keepalive = None

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._L.fasted_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- dataset ---------------------------------------------------------
    def set_points(self, pts: np.ndarray, d: int | None = None) -> None:
        """pts: (n, ld) binary16 (dtype float16 or uint16 bit patterns) on the host."""
        if pts.dtype == np.float16:
            pts = pts.view(np.uint16)
        assert pts.dtype == np.uint16 and pts.ndim == 2
        pts = np.ascontiguousarray(pts)
        n, ld = pts.shape
        d = ld if d is None else d
        _check(self._L.fasted_set_points_host_f16(self._h, pts.ctypes.data_as(_vp), n, d, ld))

    def set_points_ptr(self, host_ptr: int, n: int, d: int, ld: int) -> None:
        """Raw host pointer variant (e.g. a pinned torch tensor's data_ptr())."""
        _check(self._L.fasted_set_points_host_f16(self._h, _vp(host_ptr), n, d, ld))

    def set_points_device(self, dev_ptr: int, n: int, d: int, ld: int, keepalive=None) -> None:
        self._keepalive = keepalive
        _check(self._L.fasted_set_points_device_f16(self._h, _vp(dev_ptr), n, d, ld))

    def generate_exponential(self, n: int, d: int, lam: float = 40.0, max_value: float = 10.0,
                             seed: int = 2137834274) -> None:
        _check(self._L.fasted_generate_exponential(self._h, n, d, lam, max_value, seed))

    def fill_exponential_device(self, dev_ptr: int, n: int, d: int, ld: int, lam: float = 40.0,
                                max_value: float = 10.0, seed: int = 2137834274) -> None:
        _check(self._L.fasted_fill_exponential_device(self._h, _vp(dev_ptr), n, d, ld, lam, max_value, seed))

    def copy_points_from(self, other: "SelfJoin") -> None:
        """Replicate another context's resident dataset (same process, any GPU) device to device."""
        _check(self._L.fasted_copy_points_from(self._h, other._h))

    def set_stream(self, cuda_stream: int) -> None:
        _check(self._L.fasted_set_stream(self._h, _vp(cuda_stream)))

    def points_info(self) -> tuple[int, int, int, int]:
        dev, n, d, ld = _vp(), _i64(), _i64(), _i64()
        _check(self._L.fasted_points_info(self._h, ctypes.byref(dev), ctypes.byref(n), ctypes.byref(d),
                                          ctypes.byref(ld)))
        return int(dev.value or 0), n.value, d.value, ld.value

    def get_points(self) -> np.ndarray:
        _, n, d, _ = self.points_info()
        out = np.empty((n, d), dtype=np.uint16)
        _check(self._L.fasted_get_points_host_f16(self._h, out.ctypes.data_as(_vp), d))
        return out

    def get_rows(self, rows) -> np.ndarray:
        """Selected rows of the resident dataset as binary16 bit patterns (len(rows), d)."""
        _, _, d, _ = self.points_info()
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        out = np.empty((len(rows), d), dtype=np.uint16)
        _check(self._L.fasted_get_rows_host_f16(self._h, rows.ctypes.data_as(_vp), len(rows),
                                                out.ctypes.data_as(_vp), d))
        return out

    def get_points_into(self, host_ptr: int, ld_host: int) -> None:
        _check(self._L.fasted_get_points_host_f16(self._h, _vp(host_ptr), ld_host))

    # -- compute ---------------------------------------------------------
    def row_norms(self) -> tuple[np.ndarray, float]:
        ms = ctypes.c_double()
        _check(self._L.fasted_row_norms(self._h, ctypes.byref(ms)))
        _, n, _, _ = self.points_info()
        out = np.empty(n, dtype=np.float32)
        _check(self._L.fasted_get_norms(self._h, out.ctypes.data_as(_vp)))
        return out, ms.value

    def row_norms_timed(self) -> float:
        ms = ctypes.c_double()
        _check(self._L.fasted_row_norms(self._h, ctypes.byref(ms)))
        return ms.value

    def join(self, eps: float, q_begin: int = 0, q_end: int = -1, capacity: int = 0, flags: int = 0) -> JoinStats:
        st = JoinStats()
        _check(self._L.fasted_join(self._h, float(eps), q_begin, q_end, capacity, flags, ctypes.byref(st)))
        self._last = st
        self._last_dist = bool(flags & JOIN_DIST2)
        return st

    def join_stream(self, eps: float, q_begin: int = 0, q_end: int = -1, capacity: int = 0, flags: int = 0,
                    pairs_host: int = 0, dist2_host: int = 0, host_capacity: int = 0, on_chunk=None) -> JoinStats:
        """fasted_join_stream: the join with sort and device-to-host copy pipelined behind it.
        pairs_host / dist2_host are raw host addresses (e.g. a pinned tensor's data_ptr()) or 0;
        on_chunk(pairs (m, 2) int32, dist2 (m,) float32 or None, first) sees every run of records (views that
        are valid during the call only when no destination buffer was given)."""
        st = JoinStats()
        want_dist = bool(flags & JOIN_DIST2)

        def trampoline(_user, pairs_ptr, dist_ptr, first, count):
            try:
                pr = np.ctypeslib.as_array(ctypes.cast(pairs_ptr, ctypes.POINTER(ctypes.c_int32)), shape=(count, 2))
                d2 = (np.ctypeslib.as_array(ctypes.cast(dist_ptr, ctypes.POINTER(ctypes.c_float)), shape=(count,))
                      if dist_ptr and want_dist else None)
                return int(on_chunk(pr, d2, int(first)) or 0)
            except Exception as exc:  # noqa: BLE001 - reported after the call returns
                self._chunk_error = exc
                return 1

        self._chunk_error = None
        cb = CHUNK_FN(trampoline) if on_chunk is not None else ctypes.cast(None, CHUNK_FN)
        rc = self._L.fasted_join_stream(self._h, float(eps), q_begin, q_end, capacity, flags, _vp(pairs_host or None),
                                        _vp(dist2_host or None), host_capacity, cb, None, ctypes.byref(st))
        if self._chunk_error is not None:
            raise self._chunk_error
        _check(rc)
        self._last = st
        self._last_dist = want_dist
        return st

    def join_stream_shared(self, eps: float, table_address: int, capacity: int = 0, flags: int = 0,
                           pairs_host: int = 0, host_capacity: int = 0) -> JoinStats:
        """fasted_join_stream_shared: this rank's part of a join whose chunks all ranks of the node take from
        one shared table (fasted_b200.dist.SharedChunkTable); records go to their final place in the host
        buffer all ranks share.  Returns this rank's statistics."""
        st = JoinStats()
        _check(self._L.fasted_join_stream_shared(self._h, float(eps), capacity, flags, _vp(table_address),
                                                 _vp(pairs_host or None), host_capacity, ctypes.byref(st)))
        self._last = st
        self._last_dist = False
        return st

    def join_stream_arriving(self, eps: float, table_address: int, arrival: "Arrival", capacity: int = 0, flags: int = 0,
                             pairs_host: int = 0, host_capacity: int = 0) -> JoinStats:
        """fasted_join_stream_arriving: like join_stream_shared, started while the dataset is still arriving
        piece by piece (`arrival` carries one CUDA event per piece)."""
        st = JoinStats()
        _check(self._L.fasted_join_stream_arriving(self._h, float(eps), capacity, flags, _vp(table_address),
                                                   ctypes.byref(arrival), _vp(pairs_host or None), host_capacity,
                                                   ctypes.byref(st)))
        self._last = st
        self._last_dist = False
        return st

    def estimate_epsilon(self, target_mean_neighbours: float, sample_rows: int = 0, rel_tol: float = 0.01):
        """(epsilon, mean neighbours on the sample) for a target mean neighbour count per point."""
        eps, got = ctypes.c_double(), ctypes.c_double()
        _check(self._L.fasted_estimate_epsilon(self._h, float(target_mean_neighbours), sample_rows, rel_tol,
                                               ctypes.byref(eps), ctypes.byref(got)))
        return eps.value, got.value

    def join_symmetric_shard(self, eps: float, shard_rank: int, shard_world: int, capacity: int = 0,
                             flags: int = 0) -> JoinStats:
        st = JoinStats()
        _check(self._L.fasted_join_symmetric_shard(self._h, float(eps), shard_rank, shard_world, capacity, flags,
                                                   ctypes.byref(st)))
        self._last = st
        self._last_dist = bool(flags & JOIN_DIST2)
        return st

    def pairs(self, with_dist2: bool = False):
        st = self._last
        m = int(st.pairs_stored)
        pairs = np.empty((m, 2), dtype=np.int32)
        d2 = np.empty(m, dtype=np.float32) if with_dist2 else None
        _check(self._L.fasted_get_pairs(self._h, 0, m, pairs.ctypes.data_as(_vp),
                                        d2.ctypes.data_as(_vp) if with_dist2 else None))
        return (pairs, d2) if with_dist2 else pairs

    def pairs_device(self) -> tuple[int, int]:
        """Device addresses of the last join's results: (int2 (query, candidate) records, float distances or 0)."""
        p, d2 = _vp(), _vp()
        _check(self._L.fasted_pairs_device(self._h, ctypes.byref(p), ctypes.byref(d2)))
        return int(p.value or 0), int(d2.value or 0)

    def pairs_into(self, host_ptr: int, count: int) -> None:
        _check(self._L.fasted_get_pairs(self._h, 0, count, _vp(host_ptr), None))

    def brute_force_counts(self, rows, eps: float) -> np.ndarray:
        rows = np.ascontiguousarray(rows, dtype=np.int32)
        out = np.zeros(len(rows), dtype=np.uint64)
        _check(self._L.fasted_brute_force_f64(self._h, rows.ctypes.data_as(_vp), len(rows), float(eps),
                                              out.ctypes.data_as(_vp)))
        return out

    def brute_force_pairs(self, rows, eps: float, capacity: int) -> tuple[np.ndarray, np.ndarray]:
        """FP64 direct-form neighbours of the given query rows: (counts per row, sorted int32 pairs (m, 2))."""
        rows = np.ascontiguousarray(rows, dtype=np.int32)
        counts = np.zeros(len(rows), dtype=np.uint64)
        keys = np.empty(capacity, dtype=np.uint64)
        nk = ctypes.c_ulonglong()
        _check(self._L.fasted_brute_force_f64_pairs(self._h, rows.ctypes.data_as(_vp), len(rows), float(eps),
                                                    counts.ctypes.data_as(_vp), keys.ctypes.data_as(_vp), capacity,
                                                    ctypes.byref(nk)))
        if nk.value > capacity:
            raise FastedError(EINVAL, f"{nk.value} neighbours found, capacity {capacity}")
        k = np.sort(keys[: nk.value])
        pairs = np.stack([(k >> np.uint64(32)).astype(np.int32), (k & np.uint64(0xFFFFFFFF)).astype(np.int32)], 1)
        return counts, pairs

    def selftest_wait_timeout(self, limit_ms: float) -> tuple[int, float]:
        """(status bits, milliseconds waited) of the bounded-wait self-test kernel."""
        status, waited = ctypes.c_ulonglong(), ctypes.c_double()
        _check(self._L.fasted_selftest_wait_timeout(self._h, float(limit_ms), ctypes.byref(status),
                                                    ctypes.byref(waited)))
        return int(status.value), waited.value

    def set_option(self, name: str, value: int) -> None:
        _check(self._L.fasted_set_option(self._h, name.encode(), value))
