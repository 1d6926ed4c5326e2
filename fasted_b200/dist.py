"""Query-band sharding of the self-join over the GPUs of one node.

One process per GPU (torch.distributed).  The FP16 candidate matrix is replicated by ONE
broadcast from rank 0 (NCCL over NVLink when the tensors are CUDA tensors); after that the
bands are independent: rank r joins query rows [r*B, (r+1)*B) against all N candidates, and
because bands are contiguous in the query index, concatenating the per-rank sorted pair lists
in rank order gives the global row-major order the reference produces on one GPU
(source/pair.cuh:39-45 of the reference).  No other collective is on the data path; the
pair counts are summed with a scalar all-reduce.
"""
from __future__ import annotations

from typing import Callable, Protocol

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

    def join_band(self, eps: float, q_begin: int, q_end: int):
        n = self.sj.points_info()[1]
        st = self.sj.join(eps, q_begin=q_begin, q_end=q_end, capacity=max(1, (q_end - q_begin)) * 256
                          if q_end - q_begin < n else 0, flags=self.flags)
        self.last_stats = st
        return self.sj.pairs(), int(st.pairs_found)


    def join_symmetric_shard(self, eps: float, rank: int, world: int):
        st = self.sj.join_symmetric_shard(eps, rank, world, flags=self.flags)
        self.last_stats = st
        return self.sj.pairs(), int(st.pairs_found)


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


def sharded_self_join(engine: BandEngine, n: int, eps: float, gather: bool = True):
    """Join this rank's band; returns (pairs, found_total, stored_local).

    With gather=True rank 0 receives the concatenation of all bands (row-major order) and the
    other ranks their own band; found_total is the sum over ranks on every rank."""
    import torch
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        world, rank = dist.get_world_size(), dist.get_rank()
    else:
        world, rank = 1, 0
    begin, end = band_bounds(n, world, rank)
    if world == 1:
        pairs, found = engine.join_band(eps, begin, end)
        return pairs, found, len(pairs)
    # A rank whose join fails must not leave the others waiting in the next collective: the error
    # is caught, reported through the same all-reduce as the counts, and raised on every rank.
    error = None
    try:
        pairs, found = engine.join_band(eps, begin, end)
    except Exception as exc:  # noqa: BLE001 - reported to all ranks below
        error, pairs, found = exc, np.empty((0, 2), dtype=np.int32), 0
    backend = dist.get_backend()
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    t = torch.tensor([found, 1 if error is not None else 0], dtype=torch.int64, device=dev)
    dist.all_reduce(t)
    found_total, failed = int(t[0].item()), int(t[1].item())
    if failed:
        raise BandJoinError(f"the band join failed on {failed} of {world} ranks"
                            + (f"; this rank ({rank}): {error}" if error is not None else "")) from error
    stored_local = len(pairs)
    if gather:
        parts = [None] * world if rank == 0 else None
        dist.gather_object(pairs, parts, dst=0)
        if rank == 0:
            pairs = np.concatenate(parts) if parts else pairs
    return pairs, found_total, stored_local


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
    try:
        pairs, found = engine.join_symmetric_shard(eps, rank, world)
    except Exception as exc:  # noqa: BLE001 - reported to all ranks before the exchange
        error, pairs, found = exc, np.empty((0, 2), dtype=np.int32), 0
    backend = dist.get_backend()
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    t = torch.tensor([found, 1 if error is not None else 0], dtype=torch.int64, device=dev)
    dist.all_reduce(t)
    found_total, failed = int(t[0].item()), int(t[1].item())
    if failed:
        raise BandJoinError(f"the shard join failed on {failed} of {world} ranks"
                            + (f"; this rank ({rank}): {error}" if error is not None else "")) from error

    # records are sorted by (query, candidate): the destination ranges are contiguous slices
    bounds = [band_bounds(n, world, r) for r in range(world)]
    cuts = np.searchsorted(pairs[:, 0], [b for b, _ in bounds] + [n], side="left")
    send_counts = [int(cuts[r + 1] - cuts[r]) for r in range(world)]
    sc = torch.tensor(send_counts, dtype=torch.int64, device=dev)
    rc = torch.empty(world, dtype=torch.int64, device=dev)
    dist.all_to_all_single(rc, sc)
    recv_counts = [int(x) for x in rc.tolist()]
    send = torch.from_numpy(np.ascontiguousarray(pairs).reshape(-1)).to(dev)
    recv = torch.empty(2 * sum(recv_counts), dtype=torch.int32, device=dev)
    dist.all_to_all_single(recv, send, output_split_sizes=[2 * c for c in recv_counts],
                           input_split_sizes=[2 * c for c in send_counts])
    mine = recv.view(-1, 2)
    key = (mine[:, 0].to(torch.int64) << 32) | mine[:, 1].to(torch.int64)
    order = torch.argsort(key)
    mine = mine[order].cpu().numpy()

    stored_local = len(mine)
    if gather:
        parts = [None] * world if rank == 0 else None
        dist.gather_object(mine, parts, dst=0)
        if rank == 0:
            mine = np.concatenate(parts)
    return mine, found_total, stored_local
