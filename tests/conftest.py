import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def engine():
    """One engine on cuda:0 for the whole GPU test session (4 GiB arena)."""
    from gorgonia_b200 import Engine
    e = Engine(device=0, arena_bytes=4 << 30)
    yield e
    e.Close()


@pytest.fixture()
def fresh(engine):
    """The session engine with an empty arena."""
    engine.ResetAllocator()
    yield engine
    engine.Signal()
    engine.ResetAllocator()
