import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device; run with -m gpu")


@pytest.fixture(scope="session")
def oracle_mod():
    """The CPU oracle (checker only)."""
    import oracle
    oracle.build()
    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def native_lib():
    """The product's native library; built in-tree if missing."""
    from fasted_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from fasted_b200 import build
        build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def gpu_join(native_lib):
    """One SelfJoin context on cuda:0 for the whole GPU session."""
    from fasted_b200 import SelfJoin
    sj = SelfJoin(0)
    yield sj
    sj.close()
