import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import sm_oracle

    sm_oracle.build()
    return sm_oracle


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device and the compiled library; none is visible")
    from sharpmind_b200 import ops

    ctx = ops.CudaContext(0)
    yield ctx
    try:
        assert ctx.device_status() == 0  # no kernel abandoned a bounded wait during the session
    finally:
        ctx.close()


@pytest.fixture(scope="session")
def dev(cuda):
    from sharpmind_b200 import ops

    return ops.DeviceOps(cuda)
