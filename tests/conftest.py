import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture
def device_ok():
    """After a GPU test: the kernels must not have abandoned any bounded wait."""
    yield
    from triton_flashattn_b200 import _cabi

    st = _cabi.device_status(0)
    if st[0] != 0:
        _cabi.reset_device_status(0)
        pytest.fail(f"device status word reports an abandoned wait: {st}")
