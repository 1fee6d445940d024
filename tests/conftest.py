import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def built():
    """The swap library and the CPU checker, built in place when missing."""
    import __graft_entry__ as entry
    from torpor_b200 import _cabi
    from oracle import tso
    if not os.path.exists(_cabi.LIB_PATH) or not tso.available("oracle"):
        entry.build()
    return True


@pytest.fixture(scope="session")
def oracle_backend(built):
    import scenarios
    return scenarios.TsoBackend("oracle")


@pytest.fixture(scope="session")
def ref_backend(built):
    """The reference's own headers over the host-memory CUDA stand-in, when that
    checker has been built (it needs the reference tree at build time)."""
    from oracle import tso
    import scenarios
    if not tso.available("ref_fake"):
        pytest.skip("oracle/_ref/libtorpor_ref_fake.so not built (reference tree absent)")
    return scenarios.TsoBackend("ref_fake")
