"""pytest configuration: the `gpu` marker and shared helpers."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu")


@pytest.fixture(scope="session")
def rt():
    """The CUDA runtime mirror, initialised on cuda:0.  Fails (never skips) if the
    library is missing: there is no CPU implementation behind it."""
    import torch

    assert torch.cuda.is_available(), "gpu tests need a CUDA device"
    from reinstinct_b200 import runtime

    torch.cuda.set_device(0)
    runtime.init(0)
    return runtime
