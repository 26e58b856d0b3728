import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """Make sure the product library and the C oracle exist (both compile without a GPU)."""
    from ruy_b200 import build as b
    b.build()
    import oracle
    if not os.path.exists(oracle.ORACLE_SO):
        oracle.build(want_reference=False)


@pytest.fixture(scope="session")
def gpu_ctx():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.init()
    import ruy_b200
    ctx = ruy_b200.Context(0)
    yield ctx
    ctx.close()
