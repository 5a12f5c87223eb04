"""Copy-engine put / get / put+signal between 2 GPUs (csrc/shmem/shmem_kernels.cu, rocm_systems_b200/shmem.py)."""
import pytest

from test_gpu_fused_multi import _launch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def test_copy_engine_put_get_signal():
    _launch(2, 29871, "shmem_dma_worker.py", timeout=600)
