"""Two real GPUs (skipped on a single-GPU box): band sharding and the symmetric shard exchange over
NCCL give the same global pair list as one GPU."""
import os
import socket
import sys

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, d, eps, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from fasted_b200 import SelfJoin, _lib
    from fasted_b200.dist import GpuBandEngine, broadcast_points, sharded_self_join, sharded_self_join_symmetric
    t = torch.zeros((n, d), dtype=torch.float16, device="cuda")
    if rank == 0:
        host = _lib.dataset_exponential(n, d)
        t.copy_(torch.from_numpy(host.view(np.float16)))
    broadcast_points(t)  # the one collective of the full schedule
    sj = SelfJoin(rank)
    sj.set_points_device(t.data_ptr(), n, d, d, keepalive=t)
    sj.set_option("band_tiles", 2)
    sj.set_option("query_stationary", 0)  # raster bands of 2 tile rows: two dozen chunks to deal out
    eng = GpuBandEngine(sj)
    a, fa, _ = sharded_self_join(eng, n, eps)
    b, fb, _ = sharded_self_join_symmetric(eng, n, eps)
    # chunks taken on demand from the shared table, every chunk copied to its final place in ONE shared host list
    from fasted_b200.dist import SharedChunkTable, SharedPairBuffer, dealt_self_join
    table = SharedChunkTable.collective(n)
    shared = SharedPairBuffer.collective(fa + 100, register_cuda=True)
    fc, sc, st = dealt_self_join(sj, n, eps, table, shared, capacity=fa + 100)
    dealt_list = shared.array[:sc].copy()
    shared.array[:] = -1
    fd, sd, st2 = dealt_self_join(sj, n, eps, table, None, capacity=fa + 100, flags=_lib.JOIN_NO_SORT)
    # the same join started while the matrix is still arriving: every rank holds its band on the host, uploads
    # and all-gathers it in two pieces on side streams, and joins its first chunks behind the pieces' events
    from fasted_b200.dist import band_rows, load_and_join
    pieces = 2
    per = band_rows(n, world, 256 * pieces)
    big = torch.zeros((world * per, d), dtype=torch.float16, device="cuda")
    host_band = torch.zeros((per, d), dtype=torch.float16).pin_memory()
    mine = t[rank * per:min(n, (rank + 1) * per)]
    host_band[:mine.shape[0]].copy_(mine)
    torch.cuda.synchronize()
    fe, se, st3 = load_and_join(sj, big, host_band, n, d, eps, table, shared, capacity=fa + 100, pieces=pieces)
    arriving = shared.array[:se].copy()
    loaded_ok = bool(torch.equal(big[:n], t))
    if rank == 0:
        np.save(os.path.join(out_dir, "arriving.npy"), arriving)
        np.save(os.path.join(out_dir, "arriving_counts.npy"), np.array([fe, se, int(loaded_ok)]))
        np.save(os.path.join(out_dir, "bands.npy"), a)
        np.save(os.path.join(out_dir, "sym.npy"), b)
        np.save(os.path.join(out_dir, "dealt.npy"), dealt_list)
        np.save(os.path.join(out_dir, "found.npy"), np.array([fa, fb, fc, sc, fd]))
    np.save(os.path.join(out_dir, f"chunks{rank}.npy"), np.array([st.chunks, st2.chunks]))
    dist.barrier()
    shared.close()
    table.close()
    dist.barrier()
    sj.close()
    dist.destroy_process_group()


def test_two_gpu_sharding_matches_one_gpu(gpu_join, oracle_mod, tmp_path):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    n, d, eps = 6000, 128, 0.33
    mp.spawn(_worker, args=(2, _free_port(), n, d, eps, str(tmp_path)), nprocs=2, join=True)
    gpu_join.set_points(oracle_mod.gen_exponential(n, d))
    gpu_join.join(eps)
    want = gpu_join.pairs()
    assert np.array_equal(np.load(tmp_path / "bands.npy"), want)
    assert np.array_equal(np.load(tmp_path / "sym.npy"), want)
    assert np.array_equal(np.load(tmp_path / "dealt.npy"), want)
    assert list(np.load(tmp_path / "found.npy")) == [len(want)] * 5
    assert np.array_equal(np.load(tmp_path / "arriving.npy"), want)
    assert list(np.load(tmp_path / "arriving_counts.npy")) == [len(want), len(want), 1]
    chunks = [np.load(tmp_path / f"chunks{r}.npy") for r in range(2)]
    assert chunks[0][0] + chunks[1][0] == chunks[0][1] + chunks[1][1] >= 20  # every chunk taken exactly once, both times
