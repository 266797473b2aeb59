"""Shared fixtures.  Tests marked `gpu` are the parity tests proper: they call the CUDA path
through the C ABI and compare with the CPU oracle.  Everything else runs without a GPU."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) device")


@pytest.fixture(scope="session")
def be():
    """One backend context on cuda:0 for the whole session.  No fallback: a missing library or
    device is an error, not a skip."""
    from fandhe_ai_b200 import Backend

    b = Backend(0)
    yield b
    b.close()


@pytest.fixture()
def fresh_be():
    from fandhe_ai_b200 import Backend

    b = Backend(0)
    yield b
    b.close()
