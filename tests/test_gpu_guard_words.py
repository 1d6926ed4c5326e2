"""Guard words around caller-owned buffers: the kernels must never write outside what they were given.
(A memory checker is not available on the test machines; the reference's own safeguard is the
capacity test in its pair append, source/pair.cuh:123-133 of the reference.)  The pair buffer handed
to the join is followed by a block of pattern words; overflowing joins, ragged shapes and capacities
that are not multiples of anything must leave the pattern untouched and fill exactly `stored` slots."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

PATTERN = -0x0123456789ABCDF  # any value that is not a valid record


@pytest.mark.parametrize("n,d,eps,capacity", [
    (1000, 64, 0.25, 777),       # overflow: far more hits than slots
    (1000, 64, 0.25, 1),         # a single slot
    (3001, 200, 0.36, 4099),     # ragged n and d, odd capacity
    (130, 333, 1e3, 130 * 130 - 1),  # every entry hits, one slot short
    (130, 333, 1e3, 130 * 130),      # exactly full
    (4096, 128, 0.3136, 200_000),    # room to spare: the tail AND the unused slots stay untouched
    (257, 8, 1e3, 5000),
])
def test_join_never_writes_past_the_pair_buffer(native_lib, oracle_mod, n, d, eps, capacity):
    import torch
    from fasted_b200 import _lib
    rng = np.random.default_rng(n * 31 + d)
    ld = -(-d // 8) * 8
    host = np.zeros((n, ld), dtype=np.uint16)
    host[:, :d] = oracle_mod.double_to_half(rng.exponential(1 / 40.0, size=(n, d)))
    # guard rows around the points as well (they are only read; this keeps the layout honest)
    dev = torch.from_numpy(host.view(np.int16)).cuda()
    guard = 64
    out = torch.full((capacity + guard,), PATTERN, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    found, stored = _lib.join_static_scratch(dev.data_ptr(), n, d, ld, eps, out.data_ptr(), capacity)
    got = out.cpu().numpy()
    assert stored == min(found, capacity)
    assert (got[capacity:] == PATTERN).all(), "the join wrote past the capacity it was given"
    assert (got[stored:capacity] == PATTERN).all(), "slots beyond `stored` were written"
    keys = got[:stored].view(np.uint64)
    q, c = (keys >> np.uint64(32)).astype(np.int64), (keys & np.uint64(0xFFFFFFFF)).astype(np.int64)
    assert (q >= 0).all() and (q < n).all() and (c >= 0).all() and (c < n).all()  # never a padding index
    assert len(np.unique(keys)) == stored
    want, _ = oracle_mod.join_fp16_fp32(np.ascontiguousarray(host[:, :d]), eps)
    assert found == len(want)
    assert np.isin(keys, oracle_mod.pair_keys(want)).all()
