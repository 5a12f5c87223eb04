import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


@pytest.fixture(scope="session", autouse=True)
def _native_built():
    """Every test may load the native library; build it once (incremental, no GPU needed)."""
    from rocm_systems_b200.utils import build

    build.build_lib()
    yield


def gpu_count() -> int:
    try:
        import torch

        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0
