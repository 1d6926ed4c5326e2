"""The multi-rank band-sharding logic on CPU ranks (gloo, world size 2 and 3).  The join engine
is injected: here the CPU oracle stands in for the GPU so that the host-side logic -- band
bounds, the broadcast, the count reduction and the ordered gather -- is what is under test."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def test_band_bounds_cover_and_align():
    from fasted_b200.dist import band_bounds
    for n in [0, 1, 127, 128, 129, 1000, 4096, 100_000, 1_000_000]:
        for world in [1, 2, 3, 4, 8]:
            bands = [band_bounds(n, world, r) for r in range(world)]
            assert bands[0][0] == 0 and bands[-1][1] == n
            for (a, b), (c, d) in zip(bands, bands[1:]):
                assert b == c and a <= b
            for a, b in bands:
                assert a % 128 == 0 or a == n
            sizes = [b - a for a, b in bands if b > a]
            if n >= 128 * world:
                assert max(sizes) - min(sizes) <= 128 * world
    with pytest.raises(ValueError):
        band_bounds(10, 2, 2)


def test_weighted_band_bounds_follow_the_rates():
    from fasted_b200.dist import weighted_band_bounds
    for n in [0, 1, 129, 1000, 100_000, 1_000_000]:
        for w in [[1.0], [1, 1], [3, 1], [1.0, 1.1, 0.9, 1.0], [1, 0, 2], [0, 0, 0], [5, 4, 6, 5, 5, 5, 4.5, 5.5]]:
            bands = weighted_band_bounds(n, w)
            assert len(bands) == len(w) and bands[0][0] == 0 and bands[-1][1] == n
            for (a, b), (c, d) in zip(bands, bands[1:]):
                assert b == c and a <= b
            assert all(a % 128 == 0 or a == n for a, _ in bands)
            if n >= 100_000 and sum(w) > 0:
                for (a, b), x in zip(bands, w):
                    assert abs((b - a) - n * x / sum(w)) <= 256  # proportional up to tile rounding
    assert weighted_band_bounds(1000, [1, 0, 2])[1] == (384, 384)  # a stalled rank gets nothing
    with pytest.raises(ValueError):
        weighted_band_bounds(10, [])


@pytest.mark.parametrize("backing", ["shm", "memfd", "tmp"])
def test_shared_pair_buffer_is_one_mapping_for_two_openers(backing, monkeypatch):
    from fasted_b200.dist import SharedPairBuffer
    monkeypatch.setenv("FASTED_SHARED_BACKING", backing)
    a = SharedPairBuffer(1000)
    try:
        assert os.path.exists(a.path) and a.array.shape == (1000, 2)
        assert a.path.startswith({"shm": "/dev/shm/", "memfd": "/proc/", "tmp": "/"}[backing])
        b = SharedPairBuffer(1000, path=a.path)
        a.array[10:20] = np.arange(20, dtype=np.int32).reshape(10, 2)
        assert np.array_equal(b.array[10:20], a.array[10:20]) and b.address != 0
        a.unlink()
        assert not os.path.exists(a.path)
        b.array[0] = (7, 8)  # the mapping outlives the name
        assert a.array[0].tolist() == [7, 8]
        b.close()
    finally:
        a.unlink()
        a.close()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, d, eps, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from fasted_b200.dist import broadcast_points, sharded_self_join

    class OracleEngine:
        def __init__(self, pts):
            self.pts = pts

        def join_band(self, eps, a, b):
            p, _ = oracle.join_fp16_fp32(self.pts, eps, q_begin=a, q_end=b)
            return p, len(p)

        def join_symmetric_shard(self, eps, rank, world):
            # what the GPU shard emits: hits (i, j) with j >= i whose row i lies in one of the shard's
            # raster bands (band_rows query rows each, dealt out as a snake), plus their mirrors
            from fasted_b200 import _lib
            full, _ = oracle.join_fp16_fp32(self.pts, eps)
            band_rows = 128  # one tile row per band keeps several bands in this small case
            tiles = _lib.tile_schedule(len(self.pts), 0, len(self.pts), 1, 0, 128, 1, True, rank, world)
            my_rows = np.zeros(len(self.pts), dtype=bool)
            for tm in np.unique(tiles[:, 0]):
                my_rows[tm * band_rows:(tm + 1) * band_rows] = True
            up = full[(full[:, 1] >= full[:, 0]) & my_rows[full[:, 0]]]
            mir = up[up[:, 1] > up[:, 0]][:, ::-1]
            out = np.concatenate([up, mir])
            out = out[np.lexsort((out[:, 1], out[:, 0]))]
            return np.ascontiguousarray(out), len(out)

    # rank 0 owns the data, the others receive it through the one broadcast
    if rank == 0:
        t = torch.from_numpy(oracle.gen_exponential(n, d).view(np.int16).copy())
    else:
        t = torch.zeros((n, d), dtype=torch.int16)
    broadcast_points(t)
    pts = t.numpy().view(np.uint16)
    # loader variant: every rank fills only its own band, one all-gather completes the matrix
    from fasted_b200.dist import allgather_points, band_bounds, band_rows
    per = band_rows(n, world)
    full = torch.zeros((world * per, d), dtype=torch.int16)
    a, b = band_bounds(n, world, rank)
    full[a:b] = t[a:b]
    allgather_points(full, rank, world)
    # the pipelined loader (upload piece by piece, gather each piece as it lands) gives the same matrix
    from fasted_b200.dist import upload_and_allgather
    full2 = torch.zeros((world * per, d), dtype=torch.int16)
    band = torch.zeros((per, d), dtype=torch.int16)
    band[:b - a] = t[a:b]
    upload_and_allgather(full2, band, rank, world, pieces=3)
    np.save(os.path.join(out_dir, f"gathered_ok{rank}.npy"),
            np.array([torch.equal(full[:n], t), bool((full[n:] == 0).all()), torch.equal(full2, full)]))
    pairs, found, stored = sharded_self_join(OracleEngine(pts), n, eps)
    # the same with bands sized by (made-up) measured rates and a shared buffer that the caller owns
    from fasted_b200.dist import SharedPairBuffer, weighted_band_bounds
    wb = weighted_band_bounds(n, [1.0 + 0.5 * r for r in range(world)])
    shared = SharedPairBuffer.collective(found + 5)
    wpairs, wfound, wstored = sharded_self_join(OracleEngine(pts), n, eps, bounds=wb, shared=shared)
    np.save(os.path.join(out_dir, f"wpairs{rank}.npy"), np.array(wpairs))
    np.save(os.path.join(out_dir, f"wmeta{rank}.npy"), np.array([wfound, wstored, wb[rank][0], wb[rank][1]]))
    dist.barrier()
    shared.close()
    from fasted_b200.dist import sharded_self_join_symmetric
    spairs, sfound, sstored = sharded_self_join_symmetric(OracleEngine(pts), n, eps)
    np.save(os.path.join(out_dir, f"spairs{rank}.npy"), spairs)
    np.save(os.path.join(out_dir, f"smeta{rank}.npy"), np.array([sfound, sstored]))
    np.save(os.path.join(out_dir, f"pairs{rank}.npy"), pairs)
    np.save(os.path.join(out_dir, f"meta{rank}.npy"), np.array([found, stored]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_join_equals_single_rank(oracle_mod, tmp_path, world):
    n, d, eps = 700, 64, 0.2
    mp.spawn(_worker, args=(world, _free_port(), n, d, eps, str(tmp_path)), nprocs=world, join=True)
    want, _ = oracle_mod.join_fp16_fp32(oracle_mod.gen_exponential(n, d), eps)
    got = np.load(tmp_path / "pairs0.npy")
    assert np.array_equal(got, want)  # rank-order concatenation == global row-major order
    metas = [np.load(tmp_path / f"meta{r}.npy") for r in range(world)]
    assert all(np.load(tmp_path / f"gathered_ok{r}.npy").all() for r in range(world))
    assert all(int(m[0]) == len(want) for m in metas)
    assert sum(int(m[1]) for m in metas) == len(want)
    # weighted bands, caller-owned shared buffer: the same list; every rank wrote its own band only
    assert np.array_equal(np.load(tmp_path / "wpairs0.npy"), want)
    wm = [np.load(tmp_path / f"wmeta{r}.npy") for r in range(world)]
    assert all(int(m[0]) == len(want) for m in wm) and sum(int(m[1]) for m in wm) == len(want)
    assert [int(m[3] - m[2]) for m in wm] == sorted(int(m[3] - m[2]) for m in wm)  # sizes grow with the rates
    for r in range(1, world):
        p = np.load(tmp_path / f"wpairs{r}.npy")
        assert len(p) == int(wm[r][1]) and (len(p) == 0 or (p[:, 0].min() >= wm[r][2] and p[:, 0].max() < wm[r][3]))
    # symmetric schedule + all-to-all of records: same global list, every rank a contiguous range
    assert np.array_equal(np.load(tmp_path / "spairs0.npy"), want)
    smetas = [np.load(tmp_path / f"smeta{r}.npy") for r in range(world)]
    assert all(int(m[0]) == len(want) for m in smetas) and sum(int(m[1]) for m in smetas) == len(want)
    from fasted_b200.dist import band_bounds
    for r in range(1, world):
        a, b = band_bounds(n, world, r)
        sp = np.load(tmp_path / f"spairs{r}.npy")
        assert len(sp) == 0 or (sp[:, 0].min() >= a and sp[:, 0].max() < b)
    for r in range(1, world):
        a, b = band_bounds(n, world, r)
        p = np.load(tmp_path / f"pairs{r}.npy")
        assert len(p) == 0 or (p[:, 0].min() >= a and p[:, 0].max() < b)


def _failing_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    from fasted_b200.dist import BandJoinError, sharded_self_join, sharded_self_join_symmetric

    class Engine:
        """Rank 1's GPU "fails" (the native library's error surfaces as an exception on the host)."""

        def join_band(self, eps, a, b):
            if rank == 1:
                raise RuntimeError("FASTED_EKERNEL: a device-side wait ran out")
            return np.array([[a, a]], dtype=np.int32), 1

        def join_symmetric_shard(self, eps, r, w):
            if rank == 1:
                raise RuntimeError("FASTED_ECUDA: out of memory")
            return np.array([[0, 0]], dtype=np.int32), 1

    seen = []
    for fn in (sharded_self_join, sharded_self_join_symmetric):
        try:
            fn(Engine(), 512, 0.1)
            seen.append("no error")
        except BandJoinError as exc:
            seen.append(str(exc))
    # the group is still usable afterwards: every rank left the collectives in step
    t = torch.tensor([rank + 1])
    dist.all_reduce(t)
    seen.append(int(t.item()))
    with open(os.path.join(out_dir, f"seen{rank}.txt"), "w") as f:
        f.write(repr(seen))
    dist.destroy_process_group()


def test_a_failing_rank_is_reported_on_every_rank(tmp_path):
    world = 3
    mp.spawn(_failing_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        seen = eval((tmp_path / f"seen{r}.txt").read_text())
        assert seen[2] == 6
        for msg in seen[:2]:
            assert "failed on 1 of 3 ranks" in msg
            assert ("this rank (1)" in msg) == (r == 1)
    assert "device-side wait ran out" in eval((tmp_path / "seen1.txt").read_text())[0]


def _dealer(rank, world, port, out_dir):
    # Ranks take chunks from the shared table, "join" them (a deterministic number of records per chunk,
    # some of them none), publish the counts and write their records to the place the table gives.
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import time
    from fasted_b200.dist import SharedChunkTable, SharedPairBuffer
    n_rows, chunk_rows = 100_000, 256
    table = SharedChunkTable.collective(n_rows)
    pairs = SharedPairBuffer.collective(400_000)
    if rank == 0:
        assert table.init_plan(0, n_rows, chunk_rows) == -(-n_rows // chunk_rows)
    dist.barrier()
    count_of = lambda k: (k * 7919) % 11 if k % 5 else 0
    taken = []
    while True:
        k = table.take()
        if k < 0:
            break
        taken.append(k)
        if rank == 1 and len(taken) % 7 == 0:
            time.sleep(0.002)  # an uneven rank: the others simply take more chunks
        table.publish(k, count_of(k), count_of(k) + 1)
        off = table.offset(k)
        pairs.array[off:off + count_of(k)] = np.stack([np.full(count_of(k), k), np.arange(count_of(k))], 1)
    dist.barrier()
    found, stored, failed = table.totals()
    chunks = -(-n_rows // chunk_rows)
    want = np.concatenate([np.stack([np.full(count_of(k), k), np.arange(count_of(k))], 1) for k in range(chunks)])
    ok = (stored == len(want) and found == stored + chunks and failed == 0
          and np.array_equal(pairs.array[:stored], want) and table.offset(chunks) == stored)
    np.save(os.path.join(out_dir, f"dealt{rank}.npy"), np.array([int(ok), len(taken)]))
    # a rank that gives up: nobody waits for the counts it never published
    dist.barrier()
    if rank == 0:
        table.init_plan(0, n_rows, chunk_rows)
    dist.barrier()
    k = table.take()
    dist.barrier()  # everybody holds a chunk before rank 1 gives up
    seen = "none"
    if rank == 1:
        table.fail()
    else:
        table.publish(k, 1, 1)
        try:
            table.offset(chunks - 1, timeout_ms=20_000.0)
        except Exception as exc:  # noqa: BLE001
            seen = str(exc)
    with open(os.path.join(out_dir, f"dealt_fail{rank}.txt"), "w") as f:
        f.write(seen)
    dist.barrier()
    assert table.take() == -1  # a failed table hands out nothing
    pairs.close()
    table.close()
    dist.destroy_process_group()


def test_chunks_dealt_from_a_shared_table_land_in_order(native_lib, tmp_path):
    world = 3
    mp.spawn(_dealer, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res = [np.load(tmp_path / f"dealt{r}.npy") for r in range(world)]
    assert all(int(r[0]) == 1 for r in res)
    assert sum(int(r[1]) for r in res) == -(-100_000 // 256) and min(int(r[1]) for r in res) > 0
    for r in (0, 2):
        assert "gave up" in (tmp_path / f"dealt_fail{r}.txt").read_text()


@pytest.mark.parametrize("n_rows,chunk_rows,group_rows,lead", [
    (100_000, 256, 25_600, 3),   # four bands, the last partly beyond the data
    (5000, 256, 2560, 2),        # a band that ends inside a chunk
    (70_000, 4736, 35_840, 1),   # chunks that do not divide the band: its last chunk is shorter
    (9000, 512, 2560, 0),        # grouped, nothing set aside
])
def test_grouped_chunk_table_covers_every_row_once(native_lib, n_rows, chunk_rows, group_rows, lead):
    # The plan of a join that starts while the matrix arrives: every band (group) is cut into chunks from its
    # own first row, the first `lead` chunks of every band are kept for the band's own rank, the others are
    # handed out; chunk ids ascend with the rows, so the prefix of the published counts is a chunk's place.
    from fasted_b200.dist import SharedChunkTable
    table = SharedChunkTable(-(-n_rows // 128) + 65)
    try:
        chunks = table.init_plan(0, n_rows, chunk_rows, group_rows, lead)
        groups = -(-n_rows // group_rows)
        per_group = -(-group_rows // chunk_rows)
        assert chunks == groups * per_group
        ranges = [table.chunk_range(k) for k in range(chunks)]
        covered, prev_end = 0, 0
        for k, (b, e) in enumerate(ranges):
            assert prev_end <= b <= e <= n_rows
            if e > b:
                assert b == prev_end and b == (k // per_group) * group_rows + (k % per_group) * chunk_rows
                prev_end = e
            covered += e - b
        assert covered == n_rows and prev_end == n_rows
        handed = []
        while (k := table.take()) >= 0:
            handed.append(k)
        kept = [k for k in range(chunks) if k % per_group < lead]
        assert sorted(handed + kept) == list(range(chunks)) and handed == sorted(handed)
        assert table.take() == -1
        with pytest.raises(Exception):
            table.chunk_range(chunks)
        with pytest.raises(Exception):
            table.init_plan(0, n_rows, chunk_rows, group_rows, per_group + 1)
        with pytest.raises(Exception):
            table.init_plan(256, n_rows, chunk_rows, group_rows, 0)   # groups need the whole row range
    finally:
        table.close()
        table.unlink()


def _dealer_with_leads(rank, world, port, out_dir):
    # The protocol of the join that starts while the matrix arrives, on the table's primitives: every rank first
    # "joins" the lead chunks of its own band (counted under the band's first id), then takes chunks like any
    # dealer.  A chunk's place is the sum of the counts before it -- and the lead of band r lies behind every
    # chunk of the bands before it, which are joined later: its records must wait for their place without
    # holding up the rank's own later chunks (a rank that asked for the lead's place first would wait for itself).
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fasted_b200.dist import SharedChunkTable, SharedPairBuffer
    group_rows, chunk_rows, lead = 10_240, 256, 3
    n_rows = world * group_rows - 1000
    per_group = group_rows // chunk_rows
    table = SharedChunkTable.collective(n_rows)
    pairs = SharedPairBuffer.collective(600_000)
    if rank == 0:
        assert table.init_plan(0, n_rows, chunk_rows, group_rows, lead) == world * per_group
    dist.barrier()
    rows_of = lambda k: (lambda b, e: e - b)(*table.chunk_range(k))
    count_of = lambda k: rows_of(k) // 64 + (k * 7919) % 5 if rows_of(k) else 0
    records = lambda k, m: np.stack([np.full(m, k), np.arange(m)], 1)
    lead_id = rank * per_group
    lead_count = sum(count_of(lead_id + i) for i in range(lead))
    for i in range(1, lead):
        table.publish(lead_id + i, 0, 0)
    table.publish(lead_id, lead_count, lead_count)
    taken = []
    while True:
        k = table.take()
        if k < 0:
            break
        assert k % per_group >= lead
        taken.append(k)
        table.publish(k, count_of(k), count_of(k))
        off = table.offset(k)                         # needs the chunks before k only: never this rank's lead
        pairs.array[off:off + count_of(k)] = records(k, count_of(k))
    off = table.offset(lead_id)                       # everything this rank took is published: waiting is safe
    pairs.array[off:off + lead_count] = np.concatenate([records(lead_id + i, count_of(lead_id + i)) for i in range(lead)])
    dist.barrier()
    found, stored, failed = table.totals()
    chunks = world * per_group
    want = np.concatenate([records(k, count_of(k)) for k in range(chunks)])
    ok = stored == found == len(want) and failed == 0 and np.array_equal(pairs.array[:stored], want)
    np.save(os.path.join(out_dir, f"lead{rank}.npy"), np.array([int(ok), len(taken)]))
    dist.barrier()
    pairs.close()
    table.close()
    dist.destroy_process_group()


def test_lead_chunks_find_their_place_without_holding_up_the_dealing(native_lib, tmp_path):
    world = 3
    mp.spawn(_dealer_with_leads, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res = [np.load(tmp_path / f"lead{r}.npy") for r in range(world)]
    assert all(int(r[0]) == 1 for r in res)
    assert sum(int(r[1]) for r in res) == world * (10_240 // 256 - 3)
