import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pkg():
    """The product package (ctypes binding of librlcu_b200.so)."""
    import __graft_entry__ as entry
    if not os.path.exists(os.path.join(entry.PKG_DIR, "lib", "librlcu_b200.so")):
        entry.build()
    return entry.load_package()


@pytest.fixture(scope="session")
def O():
    """The CPU oracle (test-side checker)."""
    from oracle import oracle
    oracle.lib()
    return oracle
