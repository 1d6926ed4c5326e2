"""Failure detection without a GPU fault: a device-side wait that nothing completes runs into its
limit, the kernel returns an error status that the host reads, and the context stays usable."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_context_survives(gpu_join, oracle_mod):
    status, waited_ms = gpu_join.selftest_wait_timeout(50.0)
    assert status & 1, "the waiting thread must report its timeout"
    assert status & 2, "the second waiter must leave through the abort flag"
    assert 50.0 <= waited_ms < 500.0
    # the same context still computes correctly afterwards
    pts = oracle_mod.gen_exponential(1000, 64)
    gpu_join.set_points(pts)
    st = gpu_join.join(0.001)
    assert st.status == 0 and st.pairs_found == 1000
    from fasted_b200 import FastedError
    with pytest.raises(FastedError):
        gpu_join.selftest_wait_timeout(5000.0)  # limits above one second are refused
