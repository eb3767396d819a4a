import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def reference_root():
    """Root of a Gradiated/carat checkout, or None: the CARAT_REFERENCE environment variable, else
    a directory named `reference` beside this repository."""
    candidates = [os.environ.get("CARAT_REFERENCE"),
                  os.path.join(os.path.dirname(ROOT), "reference")]
    for candidate in candidates:
        if candidate and os.path.isdir(os.path.join(candidate, "include", "carat")):
            return candidate
    return None
