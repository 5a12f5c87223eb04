"""Copy-engine put / get / put+signal between 2 GPUs (csrc/shmem/shmem_kernels.cu, rocm_systems_b200/shmem.py).

Not yet passed on hardware: until it has, a failure is reported as an expected one (a pass shows as XPASS)."""
import pytest

from test_gpu_fused_multi import _launch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


@pytest.mark.xfail(reason="first run on hardware pending", strict=False)
def test_copy_engine_put_get_signal():
    _launch(2, 29871, "shmem_dma_worker.py", timeout=600)
