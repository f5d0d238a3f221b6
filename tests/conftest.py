import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def gctx():
    """One library context on cuda:0 shared by the GPU tests."""
    import grape_b200
    ctx = grape_b200.Context(0)
    yield ctx
    ctx.close()
