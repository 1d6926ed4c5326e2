"""Query-band sharding of the self-join over the GPUs of one node.

One process per GPU (torch.distributed).  The FP16 candidate matrix is replicated by ONE
broadcast from rank 0 (NCCL over NVLink when the tensors are CUDA tensors); after that the
bands are independent: rank r joins query rows [r*B, (r+1)*B) against all N candidates, and
because bands are contiguous in the query index, concatenating the per-rank sorted pair lists
in rank order gives the global row-major order the reference produces on one GPU
(source/pair.cuh:39-45 of the reference).  No other collective is on the data path; the
per-rank pair counts are exchanged with one all-gather of three integers, and the bands' lists
meet in one shared host buffer (SharedPairBuffer), each at the offset its predecessors' counts give.

Three ways to split the rows: fixed bands (sharded_self_join), chunks of raster bands taken on demand from
a table in shared host memory so that a faster GPU takes more (dealt_self_join), and the same with the join
started while the matrix is still being uploaded and all-gathered piece by piece (load_and_join).
"""
from __future__ import annotations

import ctypes
import mmap
import os
import tempfile
import uuid
from typing import Callable, Protocol, Sequence

import numpy as np

BAND_ALIGN = 128  # query rows per join tile: bands start on tile boundaries


def band_bounds(n: int, world: int, rank: int, align: int = BAND_ALIGN) -> tuple[int, int]:
    """Contiguous band of query rows owned by `rank`; bands are multiples of `align` rows
    (except the last non-empty one) and cover [0, n) without overlap."""
    if n < 0 or world < 1 or not (0 <= rank < world):
        raise ValueError("bad band arguments")
    per = -(-n // world)
    per = -(-per // align) * align
    begin = min(n, rank * per)
    end = min(n, begin + per)
    return begin, end


def weighted_band_bounds(n: int, weights: Sequence[float], align: int = BAND_ALIGN) -> list[tuple[int, int]]:
    """Contiguous bands of query rows, one per rank, whose sizes are proportional to `weights` (each
    rank's measured join rate, rows per millisecond): the job's step time is the slowest rank's, and
    GPUs under their own power caps do not run at the same clock, so equal bands leave the faster
    ones idle.  Bands start on multiples of `align` rows and cover [0, n) without overlap; a rank
    whose weight is zero or negative gets an empty band."""
    w = [max(float(x), 0.0) for x in weights]
    if n < 0 or not w:
        raise ValueError("bad band arguments")
    if sum(w) <= 0.0:
        w = [1.0] * len(w)
    units = -(-n // align)  # whole tiles to hand out
    total = sum(w)
    cuts, acc = [0], 0.0
    for x in w:
        acc += x
        cuts.append(min(units, max(cuts[-1], int(round(acc / total * units)))))
    cuts[-1] = units
    return [(min(n, a * align), min(n, b * align)) for a, b in zip(cuts, cuts[1:])]


class SharedMapping:
    """A block of host memory that every rank of the node maps.  Backing, in this order: a file under
    /dev/shm when it has room; else an anonymous memory file (memfd) that the other ranks open through
    /proc/<pid>/fd (containers often mount a tiny /dev/shm); else a file under the temporary directory.
    FASTED_SHARED_BACKING = shm | memfd | tmp forces one.  Rank 0 creates the mapping and removes its name
    (closes its descriptor) as soon as every rank has mapped it, so nothing is left behind if a rank dies later."""

    def __init__(self, nbytes: int, path: str | None = None):
        self.nbytes = max(int(nbytes), 8)
        self.created = path is None
        self._keep_fd = None
        if path is None:
            how = os.environ.get("FASTED_SHARED_BACKING", "")
            if not how:
                how = "memfd" if hasattr(os, "memfd_create") else "tmp"
                try:
                    st = os.statvfs("/dev/shm")
                    if st.f_bavail * st.f_frsize >= self.nbytes + (64 << 20):
                        how = "shm"
                except OSError:
                    pass
            if how == "memfd":
                fd = os.memfd_create("fasted_shared")
                os.ftruncate(fd, self.nbytes)
                self._keep_fd = os.dup(fd)  # the name the other ranks open lives as long as this descriptor
                path = f"/proc/{os.getpid()}/fd/{self._keep_fd}"
            else:
                root = "/dev/shm" if how == "shm" else tempfile.gettempdir()
                path = os.path.join(root, f"fasted_{os.getpid()}_{uuid.uuid4().hex}")
                fd = os.open(path, os.O_CREAT | os.O_EXCL | os.O_RDWR, 0o600)
                os.ftruncate(fd, self.nbytes)
        else:
            fd = os.open(path, os.O_RDWR)
        self.path = path
        try:
            self._mm = mmap.mmap(fd, self.nbytes)  # MAP_SHARED
        finally:
            os.close(fd)
        self.bytes = np.frombuffer(self._mm, dtype=np.uint8)
        self.address = self.bytes.ctypes.data

    def unlink(self) -> None:
        """Remove the mapping's name (the memory stays while it is mapped)."""
        if self._keep_fd is not None:
            os.close(self._keep_fd)
            self._keep_fd = None
        elif self.path and not self.path.startswith("/proc/") and os.path.exists(self.path):
            os.unlink(self.path)

    def close(self) -> None:
        if getattr(self, "_mm", None) is None:
            return
        self.bytes = None
        try:
            self._mm.close()
        except BufferError:
            pass  # a caller still holds a view; the mapping goes when the view does
        self._mm = None

    @classmethod
    def _collective(cls, make, attach):
        """Called by every rank: rank 0 creates the mapping (make()), the others map it (attach(path, nbytes))."""
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
            obj = make()
            obj.unlink()
            return obj
        rank = dist.get_rank()
        box = [None]
        obj = None
        if rank == 0:
            obj = make()
            box = [(obj.path, obj.nbytes)]
        dist.broadcast_object_list(box, src=0)
        if rank != 0:
            obj = attach(box[0][0], box[0][1])
        dist.barrier()
        if rank == 0:
            obj.unlink()
        return obj


class SharedPairBuffer(SharedMapping):
    """ONE host buffer for the whole job's pair list, mapped by every rank of the node.

    The reference's caller receives one row-major list (source/pair.cuh:39-45, 139-146 of the
    reference).  With one process per GPU the list is assembled without any copy between processes:
    every rank maps the buffer, page-locks its view with cudaHostRegister so that its GPU writes into
    it by DMA, and copies its sorted records to the place the counts of the records before them give."""

    def __init__(self, capacity_pairs: int, path: str | None = None, register_cuda: bool = False):
        self.capacity = max(int(capacity_pairs), 1)
        super().__init__(self.capacity * 8, path)
        self.array = self.bytes.view(np.int32).reshape(-1, 2)
        self.registered = False
        if register_cuda:
            import torch
            rc = torch.cuda.cudart().cudaHostRegister(self.address, self.nbytes, 0)
            self.registered = int(rc) == 0  # not registered: copies go through the library's pinned staging

    def close(self) -> None:
        if getattr(self, "_mm", None) is None:
            return
        if self.registered:
            import torch
            torch.cuda.cudart().cudaHostUnregister(self.address)
            self.registered = False
        self.array = None
        super().close()

    @classmethod
    def collective(cls, capacity_pairs: int, register_cuda: bool = False) -> "SharedPairBuffer":
        """Called by every rank: rank 0 creates the buffer, the others map it."""
        return cls._collective(lambda: cls(capacity_pairs, register_cuda=register_cuda),
                               lambda path, nbytes: cls(nbytes // 8, path=path, register_cuda=register_cuda))


class SharedChunkTable(SharedMapping):
    """The table from which the ranks of a node take their chunks of a streamed join
    (fasted_shared_chunks_* of the native library): a counter of chunks handed out and, per chunk, the
    number of records its rank stored, which gives every later chunk its place in the shared list."""

    def __init__(self, max_chunks: int, path: str | None = None, nbytes: int | None = None):
        from . import _lib
        self._L = _lib.load()
        super().__init__(nbytes if nbytes is not None else self._L.fasted_shared_chunks_bytes(max(int(max_chunks), 1)), path)

    @classmethod
    def collective(cls, n_rows: int) -> "SharedChunkTable":
        """Room for any chunking of n_rows query rows (a chunk is at least one 128-row tile row)."""
        max_chunks = -(-n_rows // BAND_ALIGN) + 65  # (+ one partly filled chunk per group of a grouped plan)
        return cls._collective(lambda: cls(max_chunks), lambda path, nbytes: cls(0, path=path, nbytes=nbytes))

    def init(self, self_join, eps: float, q_begin: int, q_end: int, ranks: int) -> int:
        """By ONE rank, before the others are let in: plan the chunks (from that rank's context) and reset the table."""
        from . import _lib
        chunks = ctypes.c_uint64()
        _lib._check(self._L.fasted_shared_chunks_init(self_join._h, ctypes.c_void_p(self.address), self.nbytes, float(eps),
                                                      q_begin, q_end, ranks, ctypes.byref(chunks)))
        return int(chunks.value)

    def init_plan(self, q_begin: int, q_end: int, chunk_rows: int, group_rows: int = 0, lead_chunks: int = 0) -> int:
        from . import _lib
        chunks = ctypes.c_uint64()
        _lib._check(self._L.fasted_shared_chunks_init_plan(ctypes.c_void_p(self.address), self.nbytes, q_begin, q_end,
                                                           chunk_rows, group_rows, lead_chunks, ctypes.byref(chunks)))
        return int(chunks.value)

    def init_arriving(self, self_join, eps: float, ranks: int, arrival) -> int:
        """By ONE rank: the plan for a join that starts while the dataset is arriving (fasted_join_stream_arriving)."""
        from . import _lib
        chunks = ctypes.c_uint64()
        _lib._check(self._L.fasted_shared_chunks_init_arriving(self_join._h, ctypes.c_void_p(self.address), self.nbytes,
                                                               float(eps), ranks, ctypes.byref(arrival), ctypes.byref(chunks)))
        return int(chunks.value)

    def chunk_range(self, chunk: int) -> tuple[int, int]:
        from . import _lib
        b, e = ctypes.c_int64(), ctypes.c_int64()
        _lib._check(self._L.fasted_shared_chunks_range(ctypes.c_void_p(self.address), chunk, ctypes.byref(b), ctypes.byref(e)))
        return int(b.value), int(e.value)

    def take(self) -> int:
        return int(self._L.fasted_shared_chunks_take(ctypes.c_void_p(self.address)))

    def publish(self, chunk: int, stored: int, found: int) -> None:
        from . import _lib
        _lib._check(self._L.fasted_shared_chunks_publish(ctypes.c_void_p(self.address), chunk, stored, found))

    def offset(self, chunk: int, timeout_ms: float = 60_000.0) -> int:
        from . import _lib
        off = ctypes.c_uint64()
        _lib._check(self._L.fasted_shared_chunks_offset(ctypes.c_void_p(self.address), chunk, float(timeout_ms),
                                                        ctypes.byref(off)))
        return int(off.value)

    def fail(self) -> None:
        self._L.fasted_shared_chunks_fail(ctypes.c_void_p(self.address))

    def totals(self) -> tuple[int, int, int]:
        """(pairs found, pairs stored, failed flag) over all ranks, once every rank is done."""
        from . import _lib
        f, s_, bad = ctypes.c_ulonglong(), ctypes.c_ulonglong(), ctypes.c_ulonglong()
        _lib._check(self._L.fasted_shared_chunks_totals(ctypes.c_void_p(self.address), ctypes.byref(f), ctypes.byref(s_),
                                                        ctypes.byref(bad)))
        return int(f.value), int(s_.value), int(bad.value)


def dealt_self_join(self_join, n: int, eps: float, table: SharedChunkTable, pairs: SharedPairBuffer | None = None,
                    capacity: int = 0, flags: int = 0):
    """The self-join over the ranks of one node with chunks dealt out on demand (see SharedChunkTable):
    faster GPUs take more chunks, and every rank copies its sorted chunks to their final place in the ONE
    shared host list `pairs` while the join runs.  Collective: every rank calls it.  With
    flags & JOIN_NO_SORT nothing is sorted or copied (a counting / timing run with the same balance).
    Returns (found_total, stored_total, this rank's JoinStats); raises BandJoinError on every rank when
    any rank failed."""
    import torch.distributed as dist
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    world = dist.get_world_size() if multi else 1
    rank = dist.get_rank() if multi else 0
    if rank == 0:
        table.init(self_join, eps, 0, n, world)
    if multi:
        dist.barrier()  # the table is ready
    error, st = None, None
    try:
        st = self_join.join_stream_shared(eps, table.address, capacity=capacity, flags=flags,
                                          pairs_host=pairs.address if pairs is not None else 0,
                                          host_capacity=pairs.capacity if pairs is not None else 0)
    except Exception as exc:  # noqa: BLE001 - the table is marked; every rank learns of it below
        error = exc
        table.fail()
    if multi:
        dist.barrier()  # every rank's chunks are in place
    found, stored, failed = table.totals()
    if failed or error is not None:
        raise BandJoinError(f"the join failed on at least one of {world} ranks"
                            + (f"; this rank ({rank}): {error}" if error is not None else "")) from error
    return found, stored, st


class BandJoinError(RuntimeError):
    """Raised on EVERY rank when the join of at least one rank's band failed."""


class BandEngine(Protocol):
    def join_band(self, eps: float, q_begin: int, q_end: int) -> tuple[np.ndarray, int]:
        """Sorted (m, 2) int32 pairs of the band and the number of pairs found."""

    def join_symmetric_shard(self, eps: float, rank: int, world: int) -> tuple[np.ndarray, int]:
        """Sorted pairs of shard `rank` of the symmetric schedule (both orientations of every hit in
        the shard's part of the upper triangle) and their number."""


class GpuBandEngine:
    """BandEngine on the native library (fasted_b200.SelfJoin)."""

    def __init__(self, self_join, flags: int = 0):
        self.sj = self_join
        self.flags = flags
        self.last_stats = None
        self.capacity_per_row = 256   # the reference's pair-buffer rule (n * 256), per band row
        self.capacity_rows = 0        # 0: size the buffer by the band; else by this many rows (stable across bands)

    def join_band(self, eps: float, q_begin: int, q_end: int):
        st = self.sj.join(eps, q_begin=q_begin, q_end=q_end,
                          capacity=max(1, self.capacity_rows or (q_end - q_begin)) * self.capacity_per_row,
                          flags=self.flags)
        self.last_stats = st
        return self.sj.pairs(), int(st.pairs_found)


    def join_band_device(self, eps: float, q_begin: int, q_end: int, capacity: int = 0):
        """Join the band and leave its sorted list on the device (the sort runs chunk by chunk behind
        the join): returns (stored, found).  copy_band_to() then places it anywhere on the host."""
        if not capacity:
            capacity = max(1, self.capacity_rows or (q_end - q_begin)) * self.capacity_per_row
        st = self.sj.join_stream(eps, q_begin=q_begin, q_end=q_end, capacity=capacity, flags=self.flags)
        self.last_stats = st
        return int(st.pairs_stored), int(st.pairs_found)

    def copy_band_to(self, host_address: int, count: int) -> None:
        self.sj.pairs_into(host_address, count)

    def join_symmetric_shard(self, eps: float, rank: int, world: int):
        st = self.sj.join_symmetric_shard(eps, rank, world, flags=self.flags)
        self.last_stats = st
        return self.sj.pairs(), int(st.pairs_found)

    def join_symmetric_shard_device(self, eps: float, rank: int, world: int):
        """The same, with the shard's sorted records left on the device: returns (an (m, 2) int32 CUDA tensor
        that aliases the library's result buffer -- valid until the next join --, pairs found)."""
        import torch
        st = self.sj.join_symmetric_shard(eps, rank, world, flags=self.flags)
        self.last_stats = st
        m = int(st.pairs_stored)
        ptr = self.sj.pairs_device()[0]

        class _View:  # the CUDA array interface lets torch wrap foreign device memory without a copy
            __cuda_array_interface__ = {"shape": (m, 2), "typestr": "<i4", "data": (ptr, False), "version": 2}

        dev = torch.device("cuda", self.sj.device)
        t = torch.as_tensor(_View(), device=dev) if m else torch.empty((0, 2), dtype=torch.int32, device=dev)
        return t, int(st.pairs_found)


def broadcast_points(points, src: int = 0):
    """The one collective of the path: replicate the FP16 matrix (a torch tensor, in place)."""
    import torch
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        # A broadcast is a byte copy: ship the matrix as bytes so that every backend takes it.
        dist.broadcast(points.view(torch.uint8), src=src)
    return points


def band_rows(n: int, world: int, align: int = BAND_ALIGN) -> int:
    """Rows per band (the same for every rank); world * band_rows(n, world) >= n."""
    per = -(-n // world)
    return -(-per // align) * align


def allgather_points(points, rank: int, world: int):
    """Loader variant for ranks that each hold their own band of the matrix: `points` is a torch
    tensor of world * band_rows rows of which rows [rank*B, (rank+1)*B) are filled on this rank; ONE
    in-place all-gather (NCCL over NVLink for CUDA tensors) fills in the rest.  It replaces the
    broadcast when the dataset reaches the GPUs over every rank's own host link instead of rank 0's."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or world == 1:
        return points
    if points.shape[0] % world:
        raise ValueError("points must hold world * band_rows rows")
    per = points.shape[0] // world
    flat = points.view(torch.uint8).reshape(-1)
    chunk = flat.numel() // world
    mine = flat[rank * chunk:(rank + 1) * chunk]
    if dist.get_backend() == "nccl":
        dist.all_gather_into_tensor(flat, mine)
    else:
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine.clone())
        for r, part in enumerate(parts):
            flat[r * chunk:(r + 1) * chunk].copy_(part)
    return points


def bind_to_gpu_numa_node(device_index: int) -> list[int] | None:
    """Pin this process to the CPU cores that are closest to its GPU (NVML's CPU affinity of the device).
    With one process per GPU on a two-socket host, page-locked host buffers allocated afterwards land
    on the GPU's own NUMA node, so the uploads of eight ranks do not all cross the socket interconnect.
    Returns the cores, or None when NVML or the affinity call is not available (nothing is changed then)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
        cores = [64 * w + b for w, mask in enumerate(words) for b in range(64) if (int(mask) >> b) & 1]
        allowed = os.sched_getaffinity(0)
        cores = [c for c in cores if c in allowed]
        if not cores:
            return None
        os.sched_setaffinity(0, cores)
        return cores
    except Exception:  # noqa: BLE001 - an optimisation only
        return None


def upload_and_allgather(points, host_band, rank: int, world: int, pieces: int = 4):
    """Loader for ranks that each hold their own band of the matrix in (pinned) HOST memory: the band is
    uploaded piece by piece on a side stream, and each piece is all-gathered (NCCL over NVLink) as soon
    as it has landed, so the host link and NVLink work at the same time instead of one after the
    other.  `points`: world * band_rows rows on the device, `host_band`: this rank's band_rows rows.
    Equivalent to copying the band into place and calling allgather_points."""
    import torch
    import torch.distributed as dist
    if points.shape[0] % world:
        raise ValueError("points must hold world * band_rows rows")
    per = points.shape[0] // world
    if host_band.shape[0] != per:
        raise ValueError("host_band must hold band_rows rows")
    mine = points[rank * per:(rank + 1) * per]
    if not (dist.is_available() and dist.is_initialized()) or world == 1:
        mine.copy_(host_band, non_blocking=True)
        return points
    pieces = max(1, min(pieces, per // BAND_ALIGN if per >= BAND_ALIGN else 1))
    cuts = [per * i // pieces // BAND_ALIGN * BAND_ALIGN for i in range(pieces)] + [per]
    on_gpu = points.is_cuda
    side = torch.cuda.Stream(device=points.device) if on_gpu else None
    events = []
    for a, b in zip(cuts, cuts[1:]):
        if on_gpu:
            with torch.cuda.stream(side):
                mine[a:b].copy_(host_band[a:b], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(side)
            events.append(ev)
        else:
            mine[a:b].copy_(host_band[a:b])
    for i, (a, b) in enumerate(zip(cuts, cuts[1:])):
        if b <= a:
            continue
        if on_gpu:
            torch.cuda.current_stream(points.device).wait_event(events[i])
        outs = [points[r * per + a:r * per + b].view(torch.uint8).reshape(-1) for r in range(world)]
        src = mine[a:b].view(torch.uint8).reshape(-1)
        dist.all_gather(outs, src.clone() if not on_gpu else src)
    return points


_loader_streams: dict = {}


def upload_and_allgather_events(points, host_band, rank: int, world: int, pieces: int = 4):
    """The same loader, entirely on side streams, for a join that starts while the matrix arrives
    (fasted_join_stream_arriving): returns one CUDA event per piece; event p completes when rows
    [g * B + p * B / P, g * B + (p + 1) * B / P) of every band g are resident on this GPU (B = band rows, a
    multiple of 256 * P).  The calling stream is not made to wait: whoever reads `points` waits for the events.
    Work enqueued on the calling stream before this call (the previous join) is waited for by the side streams."""
    import torch
    import torch.distributed as dist
    per = points.shape[0] // world
    if points.shape[0] % world or host_band.shape[0] != per:
        raise ValueError("points must hold world * band_rows rows, host_band band_rows rows")
    if per % (256 * pieces):
        raise ValueError("band rows must be a multiple of 256 * pieces")
    key = (points.device.index, "upload"), (points.device.index, "gather")
    for k in key:
        if k not in _loader_streams:
            _loader_streams[k] = torch.cuda.Stream(device=points.device)
    up, gather = _loader_streams[key[0]], _loader_streams[key[1]]
    here = torch.cuda.current_stream(points.device)
    up.wait_stream(here)
    gather.wait_stream(here)
    mine = points[rank * per:(rank + 1) * per]
    step = per // pieces
    landed = []
    with torch.cuda.stream(up):
        for p in range(pieces):
            mine[p * step:(p + 1) * step].copy_(host_band[p * step:(p + 1) * step], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(up)
            landed.append(ev)
    events = []
    multi = dist.is_available() and dist.is_initialized() and world > 1
    with torch.cuda.stream(gather):
        for p in range(pieces):
            gather.wait_event(landed[p])
            if multi:
                outs = [points[r * per + p * step:r * per + (p + 1) * step].view(torch.uint8).reshape(-1) for r in range(world)]
                dist.all_gather(outs, mine[p * step:(p + 1) * step].view(torch.uint8).reshape(-1))
            ev = torch.cuda.Event()
            ev.record(gather)
            events.append(ev)
    return events


def load_and_join(self_join, points, host_band, n: int, d: int, eps: float, table: "SharedChunkTable",
                  pairs: "SharedPairBuffer | None" = None, capacity: int = 0, flags: int = 0, pieces: int = 4,
                  lead_rows: int = 0):
    """One end-to-end step for ranks that each hold their own band of the matrix on the host: the band is uploaded
    and all-gathered piece by piece on side streams while every rank already joins the first chunks of its own
    band against the pieces that have arrived; the rest of the chunks are dealt out as in dealt_self_join.
    `points`: world * band_rows rows on the device (band_rows a multiple of 256 * pieces), rows beyond n zero.
    Collective.  Returns (found_total, stored_total, this rank's JoinStats)."""
    import torch.distributed as dist
    from . import _lib
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    world = dist.get_world_size() if multi else 1
    rank = dist.get_rank() if multi else 0
    per = points.shape[0] // world
    self_join.set_points_device(points.data_ptr(), n, d, points.shape[1], keepalive=points)  # geometry only: nothing is read
    plan = _lib.Arrival.make(pieces, world, per, rank * per, lead_rows)
    if rank == 0:
        table.init_arriving(self_join, eps, world, plan)
    if multi:
        dist.barrier()  # the table is ready (before the loader: a barrier behind it would wait for the whole load)
    events = upload_and_allgather_events(points, host_band, rank, world, pieces)
    arrival = _lib.Arrival.make(pieces, world, per, rank * per, lead_rows, [e.cuda_event for e in events])
    error, st = None, None
    try:
        st = self_join.join_stream_arriving(eps, table.address, arrival, capacity=capacity, flags=flags,
                                            pairs_host=pairs.address if pairs is not None else 0,
                                            host_capacity=pairs.capacity if pairs is not None else 0)
    except Exception as exc:  # noqa: BLE001 - the table is marked; every rank learns of it below
        error = exc
        table.fail()
    if multi:
        dist.barrier()
    found, stored, failed = table.totals()
    if failed or error is not None:
        raise BandJoinError(f"the join failed on at least one of {world} ranks"
                            + (f"; this rank ({rank}): {error}" if error is not None else "")) from error
    return found, stored, st


def _exchange_counts(dist, torch, values: list[int]) -> list[list[int]]:
    """All-gather of a few integers per rank (the only collective after the join)."""
    world = dist.get_world_size()
    backend = dist.get_backend()
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    mine = torch.tensor(values, dtype=torch.int64, device=dev)
    out = torch.empty(world * len(values), dtype=torch.int64, device=dev)
    if backend == "nccl":
        dist.all_gather_into_tensor(out, mine)
    else:
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        out = torch.cat(parts)
    return out.view(world, len(values)).tolist()


def sharded_self_join(engine: BandEngine, n: int, eps: float, gather: bool = True, bounds=None,
                      shared: SharedPairBuffer | None = None):
    """Join this rank's band; returns (pairs, found_total, stored_local).

    Every rank's sorted band list goes into ONE shared host buffer at the offset the exclusive scan of
    the per-rank counts gives (band order == global row-major order), so with gather=True rank 0 simply
    reads the whole list there; the other ranks return their own band.  found_total is the sum over
    ranks on every rank.  bounds: the ranks' bands (default: equal bands, band_bounds); shared: a
    buffer made by SharedPairBuffer.collective to reuse (default: one sized to the result, per call;
    the returned arrays are then copies)."""
    import torch
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        world, rank = dist.get_world_size(), dist.get_rank()
    else:
        world, rank = 1, 0
    begin, end = bounds[rank] if bounds is not None else band_bounds(n, world, rank)
    if world == 1:
        pairs, found = engine.join_band(eps, begin, end)
        return pairs, found, len(pairs)
    # A rank whose join fails must not leave the others waiting in the next collective: the error
    # is caught, reported through the same exchange as the counts, and raised on every rank.
    error, pairs, found, stored = None, None, 0, 0
    on_device = hasattr(engine, "join_band_device")
    try:
        if on_device:
            stored, found = engine.join_band_device(eps, begin, end)
        else:
            pairs, found = engine.join_band(eps, begin, end)
            stored = len(pairs)
    except Exception as exc:  # noqa: BLE001 - reported to all ranks below
        error, pairs, found, stored, on_device = exc, np.empty((0, 2), dtype=np.int32), 0, 0, False
    table = _exchange_counts(dist, torch, [stored, found, 1 if error is not None else 0])
    failed = sum(row[2] for row in table)
    if failed:
        raise BandJoinError(f"the band join failed on {failed} of {world} ranks"
                            + (f"; this rank ({rank}): {error}" if error is not None else "")) from error
    found_total = sum(row[1] for row in table)
    total = sum(row[0] for row in table)
    offset = sum(row[0] for row in table[:rank])
    own = shared is None
    if own:
        shared = SharedPairBuffer.collective(total, register_cuda=on_device)
    elif shared.capacity < total:
        raise ValueError(f"the shared buffer holds {shared.capacity} pairs, the result has {total}")
    if on_device:
        engine.copy_band_to(shared.address + 8 * offset, stored)
    else:
        shared.array[offset:offset + stored] = pairs
    dist.barrier()  # every band is in place
    if gather and rank == 0:
        out = shared.array[:total]
    else:
        out = shared.array[offset:offset + stored]
    if own:
        out = out.copy()
        dist.barrier()  # nobody unmaps while rank 0 still reads
        shared.close()
    return out, found_total, stored


def sharded_self_join_symmetric(engine: BandEngine, n: int, eps: float, gather: bool = True):
    """Symmetric schedule over the ranks: every unordered pair is computed once, on one rank.

    Rank r computes the raster bands r, 2G-1-r, 2G+r, ... of the upper triangle (balanced work) and
    emits both orientations, so its records can belong to any query row.  The ONE exchange step of
    this variant is an all-to-all of pair records: each rank sends every other rank the records whose
    query row lies in that rank's contiguous range (band_bounds), then sorts what it received.  After
    it, rank order concatenation is the global row-major order, exactly as in sharded_self_join.
    Returns (pairs, found_total, stored_local)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        pairs, found = engine.join_symmetric_shard(eps, 0, 1)
        return pairs, found, len(pairs)
    world, rank = dist.get_world_size(), dist.get_rank()
    error = None
    backend = dist.get_backend()
    on_device = backend == "nccl" and hasattr(engine, "join_symmetric_shard_device")
    try:
        if on_device:
            pairs, found = engine.join_symmetric_shard_device(eps, rank, world)
        else:
            pairs, found = engine.join_symmetric_shard(eps, rank, world)
    except Exception as exc:  # noqa: BLE001 - reported to all ranks before the exchange
        error, pairs, found, on_device = exc, np.empty((0, 2), dtype=np.int32), 0, False
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    t = torch.tensor([found, 1 if error is not None else 0], dtype=torch.int64, device=dev)
    dist.all_reduce(t)
    found_total, failed = int(t[0].item()), int(t[1].item())
    if failed:
        raise BandJoinError(f"the shard join failed on {failed} of {world} ranks"
                            + (f"; this rank ({rank}): {error}" if error is not None else "")) from error

    # records are sorted by (query, candidate): the destination ranges are contiguous slices
    bounds = [band_bounds(n, world, r) for r in range(world)]
    starts = [b for b, _ in bounds] + [n]
    if on_device:
        # everything stays on the GPU: cuts, the all-to-all over NVLink, and the merge of what arrives
        q = pairs[:, 0].contiguous()
        cuts = torch.searchsorted(q, torch.tensor(starts, dtype=torch.int32, device=q.device)).tolist()
        send = pairs.reshape(-1)
    else:
        cuts = np.searchsorted(pairs[:, 0], starts, side="left")
        send = torch.from_numpy(np.ascontiguousarray(pairs).reshape(-1)).to(dev)
    send_counts = [int(cuts[r + 1] - cuts[r]) for r in range(world)]
    sc = torch.tensor(send_counts, dtype=torch.int64, device=dev)
    rc = torch.empty(world, dtype=torch.int64, device=dev)
    dist.all_to_all_single(rc, sc)
    recv_counts = [int(x) for x in rc.tolist()]
    recv = torch.empty(2 * sum(recv_counts), dtype=torch.int32, device=dev)
    dist.all_to_all_single(recv, send, output_split_sizes=[2 * c for c in recv_counts],
                           input_split_sizes=[2 * c for c in send_counts])
    mine = recv.view(-1, 2)
    key = (mine[:, 0].to(torch.int64) << 32) | mine[:, 1].to(torch.int64)
    order = torch.argsort(key)
    mine = mine[order].cpu().numpy()

    stored_local = len(mine)
    if gather:
        table = _exchange_counts(dist, torch, [stored_local])
        total, offset = sum(r[0] for r in table), sum(r[0] for r in table[:rank])
        shared = SharedPairBuffer.collective(total)
        shared.array[offset:offset + stored_local] = mine
        dist.barrier()
        if rank == 0:
            mine = shared.array[:total].copy()
        dist.barrier()
        shared.close()
    return mine, found_total, stored_local
