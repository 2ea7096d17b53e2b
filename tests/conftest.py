import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with `-m gpu` on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _fresh_parallel_state():
    from slime_b200.parallel import state as mpu

    if not mpu.model_parallel_is_initialized():
        mpu.initialize_model_parallel()
    yield


@pytest.fixture(scope="session")
def kernels():
    """Build (if needed) and load the sm_100a kernel library; GPU tests fail loudly without it."""
    from slime_b200.ops import _lib, build

    build.build()
    return _lib.lib()
