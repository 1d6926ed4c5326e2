"""fasted_join_stream: the join whose sort and device-to-host copy run chunk by chunk behind the join
(the reference's serial tail is Pairs::sort -> Pairs::getPairs, source/pair.cuh:139-158 and
source/findPairs.cuh:699-716 of the reference).  Its output must be identical, record for record and
distance bit for distance bit, to fasted_join + fasted_get_pairs, whatever the chunking, the kind of
host memory and the delivery mode; the overflow rule (found counts everything, stored saturates at the
capacity) holds in total."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _points(oracle_mod, n, d, seed):
    rng = np.random.default_rng(seed)
    return oracle_mod.double_to_half(rng.exponential(1 / 40.0, size=(n, d)))


@pytest.mark.parametrize("n,d,eps,band_tiles,chunk_bands,qs,key32", [
    (4096, 128, 0.3136, 0, 0, -1, 1),   # everything automatic (one or two chunks at this size)
    (5000, 200, 0.42, 2, 1, 0, 1),      # raster kernel, 20 chunks of 256 rows, 32-bit records
    (5000, 200, 0.42, 2, 1, 0, 0),      # the same with 64-bit records
    (3001, 64, 0.2, 1, 3, 0, 1),        # ragged last chunk, d a single K step
    (9000, 1024, 1.04, 4, 2, -1, 1),
    (700, 333, 0.62, 1, 1, 0, 1),       # d not a multiple of 64
    (12_000, 200, 0.41, 0, 1, 1, 1),    # query-stationary kernel: chunks of 37 tile rows
    (12_000, 64, 0.2, 0, 1, 1, 0),
])
def test_stream_equals_join_then_get_pairs(gpu_join, oracle_mod, n, d, eps, band_tiles, chunk_bands, qs, key32):
    import torch
    pts = _points(oracle_mod, n, d, n + d)
    gpu_join.set_points(pts)
    gpu_join.set_option("band_tiles", band_tiles)
    gpu_join.set_option("stream_chunk_bands", chunk_bands)
    gpu_join.set_option("query_stationary", qs)
    gpu_join.set_option("stream_key32", key32)
    try:
        st0 = gpu_join.join(eps, flags=1)
        want, want_d2 = gpu_join.pairs(with_dist2=True)
        m = len(want)
        assert m == st0.pairs_found > n
        # (a) pinned destination, with distances
        hp = torch.full((m + 7, 2), -1, dtype=torch.int32).pin_memory()
        hd = torch.full((m + 7,), -1.0, dtype=torch.float32).pin_memory()
        seen = []
        st = gpu_join.join_stream(eps, flags=1, pairs_host=hp.data_ptr(), dist2_host=hd.data_ptr(), host_capacity=m + 7,
                                  on_chunk=lambda p, d2, first: seen.append((first, len(p), p[0].tolist(), float(d2[0]))))
        assert st.status == 0 and st.pairs_found == st.pairs_stored == m
        assert np.array_equal(hp.numpy()[:m], want) and (hp.numpy()[m:] == -1).all()
        assert np.array_equal(hd.numpy()[:m].view(np.uint32), want_d2.view(np.uint32)) and (hd.numpy()[m:] == -1).all()
        # the callback saw consecutive runs that tile [0, m), each pointing into the destination
        assert [f for f, *_ in seen] == list(np.cumsum([0] + [c for _, c, *_ in seen[:-1]]))
        assert sum(c for _, c, *_ in seen) == m
        assert all(want[f].tolist() == p0 and want_d2[f] == d0 for f, _, p0, d0 in seen)
        if chunk_bands and qs == 0:
            rows_per_chunk = chunk_bands * (band_tiles or 16) * 128
            assert st.chunks == -(-n // rows_per_chunk)
        if chunk_bands and qs == 1:
            assert st.chunks == -(-n // (chunk_bands * 37 * 128))
        assert len(seen) <= st.chunks
        # fasted_get_pairs works afterwards, as after fasted_join
        again, again_d2 = gpu_join.pairs(with_dist2=True)
        assert np.array_equal(again, want) and np.array_equal(again_d2.view(np.uint32), want_d2.view(np.uint32))
        # (b) pageable destination, no distances, no callback
        out = np.full((m, 2), -1, dtype=np.int32)
        st = gpu_join.join_stream(eps, pairs_host=out.ctypes.data, host_capacity=m)
        assert st.pairs_found == m and np.array_equal(out, want)
        # (c) callback only: the runs pass through the library's staging buffers
        got, got_d2 = [], []
        st = gpu_join.join_stream(eps, flags=1, on_chunk=lambda p, d2, first: (got.append(p.copy()), got_d2.append(d2.copy())) and 0)
        assert np.array_equal(np.concatenate(got), want)
        assert np.array_equal(np.concatenate(got_d2).view(np.uint32), want_d2.view(np.uint32))
        # (d) a band of query rows
        b0, b1 = 128, min(n, 128 + 5 * 128 + 17)
        band = np.full((m, 2), -1, dtype=np.int32)
        st = gpu_join.join_stream(eps, q_begin=b0, q_end=b1, pairs_host=band.ctypes.data, host_capacity=m)
        sel = want[(want[:, 0] >= b0) & (want[:, 0] < b1)]
        assert st.pairs_found == len(sel) and np.array_equal(band[:len(sel)], sel)
    finally:
        gpu_join.set_option("band_tiles", 0)
        gpu_join.set_option("stream_chunk_bands", 0)
        gpu_join.set_option("query_stationary", -1)
        gpu_join.set_option("stream_key32", 1)


def test_stream_against_the_oracle(gpu_join, oracle_mod):
    from util import assert_identical_to_oracle
    pts = oracle_mod.gen_exponential(3000, 192)
    gpu_join.set_points(pts)
    gpu_join.set_option("band_tiles", 2)
    gpu_join.set_option("stream_chunk_bands", 2)
    gpu_join.set_option("query_stationary", 0)  # raster bands: six chunks at this size
    try:
        got, got_d2 = [], []
        gpu_join.join_stream(0.36, flags=1, on_chunk=lambda p, d2, first: (got.append(p.copy()), got_d2.append(d2.copy())) and 0)
    finally:
        gpu_join.set_option("band_tiles", 0)
        gpu_join.set_option("stream_chunk_bands", 0)
        gpu_join.set_option("query_stationary", -1)
    assert_identical_to_oracle(oracle_mod, pts, 192, 0.36, np.concatenate(got), np.concatenate(got_d2))


def test_stream_overflow_clip_and_abort(gpu_join, oracle_mod):
    from fasted_b200 import FastedError
    pts = _points(oracle_mod, 4000, 96, 5)
    gpu_join.set_points(pts)
    gpu_join.set_option("band_tiles", 2)
    gpu_join.set_option("stream_chunk_bands", 1)
    gpu_join.set_option("query_stationary", 0)  # raster bands of 2 tile rows: chunks of 256 rows
    try:
        full = gpu_join.join(0.26)
        want = gpu_join.pairs()
        m = len(want)
        allk = oracle_mod.pair_keys(want)
        # pair buffer smaller than the result: found keeps counting, stored saturates; what is delivered
        # is sorted chunk by chunk, free of duplicates, and part of the full result
        cap = m // 3
        out = np.full((m, 2), -1, dtype=np.int32)
        st = gpu_join.join_stream(0.26, capacity=cap, pairs_host=out.ctypes.data, host_capacity=m)
        assert st.pairs_found == m and st.pairs_stored == cap
        k = oracle_mod.pair_keys(out[:cap])
        assert len(np.unique(k)) == cap and np.isin(k, allk).all() and (out[cap:] == -1).all()
        # the chunks that fitted completely come first and are exact
        whole_rows = out[:cap][:, 0].max()
        head = want[want[:, 0] < (whole_rows // 256) * 256]
        assert np.array_equal(out[:len(head)], head)
        # host buffer smaller than the result: the head of the list is copied, nothing beyond it
        small = np.full((1000 + 5, 2), -1, dtype=np.int32)
        st = gpu_join.join_stream(0.26, pairs_host=small.ctypes.data, host_capacity=1000)
        assert st.pairs_stored == m and np.array_equal(small[:1000], want[:1000]) and (small[1000:] == -1).all()
        # a callback that asks to stop: the call fails after the GPU work has drained, the context stays usable
        calls = []
        with pytest.raises(FastedError):
            gpu_join.join_stream(0.26, on_chunk=lambda p, d2, first: calls.append(first) or 1)
        assert calls == [0]
        with pytest.raises(ZeroDivisionError):
            gpu_join.join_stream(0.26, on_chunk=lambda p, d2, first: 1 // 0)
        assert gpu_join.join(0.26).pairs_found == full.pairs_found
        # flags that make no sense here are refused
        for bad in (2, 8, 16):
            with pytest.raises(FastedError):
                gpu_join.join_stream(0.26, flags=bad)
        # empty query range
        st = gpu_join.join_stream(0.26, q_begin=128, q_end=128, on_chunk=lambda *a: 1)
        assert st.pairs_found == 0
    finally:
        gpu_join.set_option("band_tiles", 0)
        gpu_join.set_option("stream_chunk_bands", 0)
        gpu_join.set_option("query_stationary", -1)


@pytest.mark.parametrize("n,d,eps,ranks", [(20_000, 128, 0.30, 2), (9000, 1024, 1.04, 3), (30_000, 64, 0.18, 4)])
def test_chunks_shared_by_several_contexts_give_the_single_list(gpu_join, oracle_mod, n, d, eps, ranks):
    # The multi-GPU form of the streamed join, here with `ranks` contexts on the GPUs that are present
    # (all on one GPU if there is only one: the kernels never wait for each other, only the host
    # threads wait for published counts): every context takes chunks from the shared table and copies
    # its sorted chunks to their final place in ONE host buffer, which must equal the one-GPU list.
    import threading
    import torch
    from fasted_b200 import SelfJoin, JOIN_NO_SORT
    from fasted_b200.dist import SharedChunkTable, SharedPairBuffer
    pts = _points(oracle_mod, n, d, 3 * n + d)
    gpu_join.set_points(pts)
    st0 = gpu_join.join(eps)
    want = gpu_join.pairs()
    assert st0.pairs_found == st0.pairs_stored == len(want) > n
    devs = torch.cuda.device_count()
    ctxs = [SelfJoin(i % devs) for i in range(ranks)]
    table = SharedChunkTable(-(-n // 128) + 1)
    pairs = SharedPairBuffer(len(want) + 64, register_cuda=True)
    try:
        for c in ctxs:
            c.set_points(pts)
            c.set_option("band_tiles", 2)           # many chunks even at this size
            c.set_option("query_stationary", 0)
        for flags in (0, JOIN_NO_SORT):
            pairs.array[:] = -1
            chunks = table.init(ctxs[0], eps, 0, n, ranks)
            assert chunks >= 4 * ranks
            stats, errors = [None] * ranks, []

            def work(i):
                try:
                    stats[i] = ctxs[i].join_stream_shared(eps, table.address, capacity=len(want) + 1000, flags=flags,
                                                          pairs_host=pairs.address, host_capacity=pairs.capacity)
                except Exception as exc:  # noqa: BLE001
                    errors.append(exc)

            threads = [threading.Thread(target=work, args=(i,)) for i in range(ranks)]
            for t in threads:
                t.start()
            for t in threads:
                t.join()
            assert not errors, errors
            found, stored, failed = table.totals()
            assert (found, stored, failed) == (len(want), len(want), 0)
            assert sum(s.chunks for s in stats) == chunks and sum(s.pairs_found for s in stats) == len(want)
            if flags == 0:
                assert np.array_equal(pairs.array[:len(want)], want) and (pairs.array[len(want):] == -1).all()
            else:
                assert (pairs.array == -1).all()  # a counting run copies nothing
    finally:
        for c in ctxs:
            c.close()
        pairs.close()
        table.close()
        pairs.unlink()
        table.unlink()


@pytest.mark.parametrize("n,d,eps,ranks,pieces,band_rows,stationary,staged", [
    (20_000, 128, 0.30, 2, 2, 10_240, 0, True),    # two bands, two pieces, the data lands behind events
    (20_000, 128, 0.30, 2, 2, 10_240, 1, True),    # query-stationary kernel (chunks of 37 tile rows: one lead chunk or none)
    (9000, 1024, 1.04, 4, 2, 2560, 0, False),      # last band partly beyond n; dataset resident already (no events)
    (30_000, 64, 0.18, 3, 1, 10_240, 0, True),     # one piece: the lead runs once, against everything
    (20_000, 128, 0.32, 2, 2, 10_240, 0, True),    # ~350 neighbours per point: the second call knows that the output
                                                   # is dense and keeps 32-bit records and one sort per chunk
])
def test_join_started_while_the_matrix_arrives(gpu_join, oracle_mod, n, d, eps, ranks, pieces, band_rows, stationary, staged):
    # fasted_join_stream_arriving with `ranks` contexts on the GPUs present.  The matrix is zero when the calls
    # start and is filled piece by piece on a side stream (piece p = rows [g*B + p*B/P, ...) of every band g),
    # one event per piece: a launch that read candidates before their event would see zeros, i.e. other pairs.
    import threading
    import torch
    from fasted_b200 import SelfJoin, _lib
    from fasted_b200.dist import SharedChunkTable, SharedPairBuffer
    pts = _points(oracle_mod, n, d, 5 * n + d)
    gpu_join.set_points(pts)
    st0 = gpu_join.join(eps, capacity=n * 512)
    want = gpu_join.pairs()
    assert st0.pairs_found == st0.pairs_stored == len(want) > n
    assert ranks * band_rows >= n and band_rows % (256 * pieces) == 0
    devs = torch.cuda.device_count()
    host = torch.zeros((ranks * band_rows, d), dtype=torch.float16).pin_memory()
    host[:n] = torch.from_numpy(pts.view(np.float16))
    ctxs, bufs, sides = [], [], []
    table = SharedChunkTable(-(-n // 128) + 65)
    pairs = SharedPairBuffer(len(want) + 64, register_cuda=True)
    try:
        for i in range(ranks):
            dev = torch.device("cuda", i % devs)
            c = SelfJoin(i % devs)
            buf = torch.zeros((ranks * band_rows, d), dtype=torch.float16, device=dev)
            c.set_points_device(buf.data_ptr(), n, d, d, keepalive=buf)
            c.set_option("band_tiles", 2)
            c.set_option("query_stationary", stationary)
            ctxs.append(c)
            bufs.append(buf)
            sides.append(torch.cuda.Stream(device=dev))
        for lead_rows in (0, 512):
            pairs.array[:] = -1
            plan = _lib.Arrival.make(pieces, ranks, band_rows, 0, lead_rows)
            chunks = table.init_arriving(ctxs[0], eps, ranks, plan)
            arrivals = []
            step = band_rows // pieces
            for i in range(ranks):
                events = None
                if staged:
                    bufs[i].zero_()
                    torch.cuda.synchronize(bufs[i].device)
                    events = []
                    with torch.cuda.stream(sides[i]):
                        for p in range(pieces):
                            torch.cuda._sleep(8_000_000)  # a few milliseconds between the pieces
                            for g in range(ranks):
                                a = g * band_rows + p * step
                                bufs[i][a:a + step].copy_(host[a:a + step], non_blocking=True)
                            ev = torch.cuda.Event()
                            ev.record(sides[i])
                            events.append(ev)
                    arrivals.append((_lib.Arrival.make(pieces, ranks, band_rows, i * band_rows, lead_rows,
                                                       [e.cuda_event for e in events]), events))
                else:
                    bufs[i].copy_(host)
                    torch.cuda.synchronize(bufs[i].device)
                    arrivals.append((_lib.Arrival.make(pieces, ranks, band_rows, i * band_rows, lead_rows), None))
            stats, errors = [None] * ranks, []

            def work(i):
                try:
                    stats[i] = ctxs[i].join_stream_arriving(eps, table.address, arrivals[i][0], capacity=len(want) + 1000,
                                                            pairs_host=pairs.address, host_capacity=pairs.capacity)
                except Exception as exc:  # noqa: BLE001
                    errors.append(exc)

            threads = [threading.Thread(target=work, args=(i,)) for i in range(ranks)]
            for t in threads:
                t.start()
            for t in threads:
                t.join()
            assert not errors, errors
            found, stored, failed = table.totals()
            assert (found, stored, failed) == (len(want), len(want), 0)
            assert sum(s.pairs_found for s in stats) == len(want)
            # every band's first chunks were joined by its own rank, as one sequence
            lead_ids = [k for k in range(chunks) if table.chunk_range(k)[0] % band_rows < 512 and lead_rows == 512]
            if lead_rows == 512:
                assert sum(s.chunks for s in stats) <= chunks - len(lead_ids) + ranks
            assert np.array_equal(pairs.array[:len(want)], want) and (pairs.array[len(want):] == -1).all()
            # a table with lead chunks cannot be joined without the arrival description
            if lead_rows == 512 and not stationary:
                table.init_arriving(ctxs[0], eps, ranks, plan)
                with pytest.raises(Exception, match="lead chunks"):
                    ctxs[0].join_stream_shared(eps, table.address, capacity=len(want) + 1000)
    finally:
        for c in ctxs:
            c.close()
        pairs.close()
        table.close()
        pairs.unlink()
        table.unlink()
