import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def backend():
    """One context on cuda:0 for the whole session.  Fails (never skips) when the CUDA library cannot be
    used: GPU tests must not pass on a fallback."""
    from slai_b200.ops import Backend
    b = Backend(0)
    yield b
    b.close()


@pytest.fixture(scope="session")
def ctx(backend):
    from slai_b200.ops import LlmContext
    return LlmContext(backend)
