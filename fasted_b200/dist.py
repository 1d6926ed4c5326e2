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


class BandEngine(Protocol):
    def join_band(self, eps: float, q_begin: int, q_end: int) -> tuple[np.ndarray, int]:
        """Sorted (m, 2) int32 pairs of the band and the number of pairs found."""


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


def broadcast_points(points, src: int = 0):
    """The one collective of the path: replicate the FP16 matrix (a torch tensor, in place)."""
    import torch
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        # A broadcast is a byte copy: ship the matrix as bytes so that every backend takes it.
        dist.broadcast(points.view(torch.uint8), src=src)
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
    pairs, found = engine.join_band(eps, begin, end)
    if world == 1:
        return pairs, found, len(pairs)
    backend = dist.get_backend()
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    t = torch.tensor([found], dtype=torch.int64, device=dev)
    dist.all_reduce(t)
    found_total = int(t.item())
    stored_local = len(pairs)
    if gather:
        parts = [None] * world if rank == 0 else None
        dist.gather_object(pairs, parts, dst=0)
        if rank == 0:
            pairs = np.concatenate(parts) if parts else pairs
    return pairs, found_total, stored_local
