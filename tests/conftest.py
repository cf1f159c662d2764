import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def port():
    import oracle
    return oracle.port()


@pytest.fixture(scope="session")
def ref():
    import oracle
    r = oracle.ref()
    if r is None:
        pytest.skip("oracle/_ref/libacl_ref.so not built (needs a Compute Library tree: make -C oracle ref)")
    return r


@pytest.fixture(scope="session")
def ctx():
    """One cugl context on cuda:0, enqueueing on torch's current stream so torch tensors can be used as
    device buffers without extra synchronisation."""
    import torch
    import computelibrary_b200 as cl
    assert torch.cuda.is_available(), "gpu-marked test run without a GPU"
    torch.cuda.set_device(0)
    c = cl.Context(0, torch.cuda.current_stream().cuda_stream)
    yield c
    c.sync()
    c.close()
