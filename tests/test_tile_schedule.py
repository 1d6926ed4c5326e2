"""The join kernel's persistent tile schedule, evaluated on the host (the same code the device runs):
every tile that must be computed is walked exactly once over all CTAs, in band-major order."""
import numpy as np
import pytest


def _all_tiles(n, q_begin, q_end, grid, tile_m, band, symmetric):
    from fasted_b200 import _lib
    per_cta = [_lib.tile_schedule(n, q_begin, q_end, grid, c, tile_m, band, symmetric) for c in range(grid)]
    return per_cta


@pytest.mark.parametrize("n,q_begin,q_end,grid,tile_m,band", [
    (1000, 0, 1000, 7, 128, 16), (5000, 0, 5000, 148, 128, 16), (5000, 1280, 3333, 148, 128, 4),
    (4096, 0, 4096, 74, 256, 8), (300, 0, 300, 148, 128, 16), (70000, 0, 70000, 148, 128, 16), (1, 0, 1, 3, 128, 1),
])
def test_full_schedule_covers_every_tile_once(native_lib, n, q_begin, q_end, grid, tile_m, band):
    per_cta = _all_tiles(n, q_begin, q_end, grid, tile_m, band, False)
    tiles_m = -(-(q_end - q_begin) // tile_m)
    tiles_n = -(-n // 256)
    allt = np.concatenate(per_cta)
    assert len(allt) == tiles_m * tiles_n
    keys = allt[:, 0].astype(np.int64) * tiles_n + allt[:, 1]
    assert len(np.unique(keys)) == len(keys) and keys.min() == 0 and keys.max() == tiles_m * tiles_n - 1
    # static round robin: CTA c takes positions c, c + grid, ... of one global order; loads differ by <= 1
    sizes = [len(t) for t in per_cta]
    assert max(sizes) - min(sizes) <= 1
    # band-major, row-fastest: the first `band` tiles of the global order share one tile column
    order = np.empty((len(allt), 2), dtype=np.int32)
    for c, t in enumerate(per_cta):
        order[c::grid][: len(t)] = t
    rows_in_band = min(band, tiles_m)
    assert (order[:rows_in_band, 1] == 0).all() and list(order[:rows_in_band, 0]) == list(range(rows_in_band))


@pytest.mark.parametrize("n,grid,tile_m,band", [(1000, 7, 128, 16), (5000, 148, 128, 16), (4096, 74, 256, 8),
                                                (70000, 148, 128, 16), (300, 5, 128, 2), (33333, 148, 128, 3)])
def test_symmetric_schedule_covers_the_upper_triangle_once(native_lib, n, grid, tile_m, band):
    per_cta = _all_tiles(n, 0, n, grid, tile_m, band, True)
    allt = np.concatenate(per_cta)
    tiles_m = -(-n // tile_m)
    tiles_n = -(-n // 256)
    tm, tn = np.meshgrid(np.arange(tiles_m), np.arange(tiles_n), indexing="ij")
    needed = (tn * 256 + 255 >= tm * tile_m)  # the tile holds an element with column >= row
    got = np.zeros((tiles_m, tiles_n), dtype=np.int32)
    np.add.at(got, (allt[:, 0], allt[:, 1]), 1)
    assert np.array_equal(got, needed.astype(np.int32))
    assert needed.sum() < 0.56 * tiles_m * tiles_n or tiles_m * tiles_n < 200


@pytest.mark.parametrize("n,world,band", [(5000, 2, 4), (70000, 8, 16), (33333, 3, 3), (300, 4, 1), (1_000_000, 8, 16)])
def test_symmetric_shards_partition_the_triangle_evenly(native_lib, n, world, band):
    from fasted_b200 import _lib
    tiles_m, tiles_n = -(-n // 128), -(-n // 256)
    got = np.zeros((tiles_m, tiles_n), dtype=np.int32)
    loads = []
    for r in range(world):
        # one "CTA" walking everything = the shard's whole tile list
        t = _lib.tile_schedule(n, 0, n, 1, 0, 128, band, True, r, world)
        np.add.at(got, (t[:, 0], t[:, 1]), 1)
        loads.append(len(t))
    tm, tn = np.meshgrid(np.arange(tiles_m), np.arange(tiles_n), indexing="ij")
    needed = (tn * 256 + 255 >= tm * 128).astype(np.int32)
    assert np.array_equal(got, needed)
    if tiles_m >= 8 * world * band:
        assert (max(loads) - min(loads)) / max(loads) < 0.02  # the snake evens out the triangle


@pytest.mark.parametrize("n,q_begin,q_end,grid,rows,symmetric", [
    (1000, 0, 1000, 7, 7, False), (5000, 0, 5000, 148, 37, False), (5000, 1280, 3333, 148, 37, False),
    (100_000, 0, 100_000, 148, 37, False), (300, 0, 300, 3, 3, False), (1, 0, 1, 1, 1, False),
    (4096, 0, 4096, 100, 25, False), (5000, 0, 5000, 148, 37, True), (33_333, 0, 33_333, 148, 37, True),
    (1000, 0, 1000, 8, 8, True), (70_000, 0, 70_000, 148, 4, False),
])
def test_stationary_schedule_covers_every_tile_once_row_by_row(native_lib, n, q_begin, q_end, grid, rows, symmetric):
    # The query-stationary kernel: every needed tile exactly once over all CTAs; a CTA walks one tile
    # row at a time (so that the row's query tile can stay in shared memory) with ascending columns;
    # the CTAs that share a row split its columns evenly.
    from fasted_b200 import _lib
    per_cta = [_lib.tile_schedule_stationary(n, q_begin, q_end, grid, c, rows, symmetric) for c in range(grid)]
    tiles_m, tiles_n = -(-(q_end - q_begin) // 128), -(-n // 256)
    tm, tn = np.meshgrid(np.arange(tiles_m), np.arange(tiles_n), indexing="ij")
    needed = (tn * 256 + 255 >= q_begin + tm * 128) if symmetric else np.ones((tiles_m, tiles_n), dtype=bool)
    got = np.zeros((tiles_m, tiles_n), dtype=np.int32)
    for t in per_cta:
        np.add.at(got, (t[:, 0], t[:, 1]), 1)
        if len(t) > 1:
            same_row = t[1:, 0] == t[:-1, 0]
            assert (t[1:, 1][same_row] > t[:-1, 1][same_row]).all()      # ascending columns inside a row
            assert (t[1:, 0][~same_row] > t[:-1, 0][~same_row]).all()    # a row is never revisited
    assert np.array_equal(got, needed.astype(np.int32))
    if not symmetric and tiles_m >= rows and tiles_n >= 4 * (grid // rows):
        full_band = [len(t[t[:, 0] < rows]) for t in per_cta if len(t)]
        assert max(full_band) - min(full_band) <= 1
    from fasted_b200 import FastedError
    with pytest.raises(FastedError):
        _lib.tile_schedule_stationary(n, q_begin, q_end, grid, 0, grid + 1, symmetric)
