import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU and the built libsdxlq.so")


@pytest.fixture(scope="session")
def pkg():
    """The package directory name contains a hyphen, so it is imported by string."""
    return importlib.import_module("sdxl-end2end_b200")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as module
    module.lib()
    return module


@pytest.fixture(scope="session")
def gpu_session(pkg):
    """(package, Context, Ops) on cuda:0. Fails loudly when the library or the GPU is missing."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    context = pkg.Context(0, workspace_bytes=1 << 30)
    ops = pkg.Ops(context, poison_outputs=True)
    yield pkg, context, ops
    context.check()
    context.close()


@pytest.fixture
def gpu(gpu_session):
    """The session's context with the tuning switches a test may have left behind put back."""
    pkg, context, ops = gpu_session
    context.set_pair_mode(0)
    context.set_tile_n(0)
    return gpu_session
