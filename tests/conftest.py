import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def cuda_device():
    """Device index for GPU tests. A GPU test on a machine without a usable device FAILS (it never falls back)."""
    import llaisys_b200 as llaisys

    n = llaisys.RuntimeAPI(llaisys.DeviceType.NVIDIA).get_device_count()
    assert n > 0, "GPU test selected but the library sees no NVIDIA device"
    import torch

    assert torch.cuda.is_available(), "GPU test selected but torch sees no CUDA device"
    torch.cuda.set_device(0)
    llaisys.set_context_runtime(llaisys.DeviceType.NVIDIA, 0)
    return 0
