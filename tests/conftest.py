import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PKG = "tensor-program-optimization-with-auto-batching_b200"


def load(sub=None):
    """The package directory name has hyphens, so it is imported by string."""
    return importlib.import_module(PKG if sub is None else f"{PKG}.{sub}")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def mlora():
    return load()


@pytest.fixture(scope="session")
def ops():
    return load("ops")


@pytest.fixture(scope="session")
def synth():
    return load("synth")


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a gpu-marked test ran without a CUDA device")
    # the C-ABI library must be the thing that runs: build it if the checkout has no binary yet
    load("build").build()
    return torch.device("cuda:0")
