import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as ge  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100); run with -m gpu on a B200")


@pytest.fixture(scope="session")
def built():
    """Builds (if stale) and loads the CUDA library and the oracle."""
    ge.build()
    return ge.load_package()


@pytest.fixture(scope="session")
def g(built):
    return built


@pytest.fixture(scope="session")
def orc(built):
    return ge.load_oracle()


@pytest.fixture(scope="session")
def gpu(g):
    """Initialised library on cuda:0. GPU tests fail loudly (never skip) without a device."""
    import torch

    assert torch.cuda.is_available(), "GPU test collected on a machine without CUDA"
    torch.cuda.set_device(0)
    g.init(0)
    return g


def golden(name):
    return np.load(os.path.join(ROOT, "tests", "golden", name))


LAYERS = ["qkv", "attn_proj", "fc", "fc_proj", "lm_head"]
