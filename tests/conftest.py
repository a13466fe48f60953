import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure): built on demand from oracle/zinc_oracle.cpp."""
    from oracle import oracle as o

    o.lib()
    return o


@pytest.fixture(scope="session")
def gpu():
    """(torch, Context, DmmvDispatch) on cuda:0, launching on torch's current stream."""
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    import zinc_b200 as zb

    torch.cuda.set_device(0)
    ctx = zb.Context(0, stream=torch.cuda.current_stream().cuda_stream)
    return torch, ctx, zb.DmmvDispatch(ctx)
