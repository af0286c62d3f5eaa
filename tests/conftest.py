import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def cdl():
    """The product package; importing it fails loudly when the CUDA library is not built."""
    import cleanlm_b200

    return cleanlm_b200


@pytest.fixture()
def gpu_ok(cdl):
    """Checks the kernel status word after each GPU test: no bounded wait may have run out."""
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    cdl._lib.check(cdl._lib.lib.cdl_b200_device_ok(0))
    yield
    assert cdl._lib.device_status() == 0, "a kernel gave up on a bounded wait"
