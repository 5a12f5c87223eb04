"""The fused tensor-parallel and expert-parallel paths on ONE GPU (a communicator of one rank): the tcgen05 GEMM with the
all-gather→GEMM policy and SwiGLU epilogue, the GEMM→reduce-scatter epilogue, staging and reducer, the expert-parallel
dispatch (route, fp8 quantise, row reservation by atomics, stores), grouped expert GEMMs and combine — all against their
plain PyTorch compositions, through the same workers the multi-GPU tests use. The collective part degenerates (nothing
crosses a link), the kernels and their schedules are the real ones.

Each runs in a child process; every device-side wait is limited to 5 s. One rank holds all experts, and the router
kernel wants a multiple of 32 of them, so the expert-parallel runs use 32 local experts."""
import pytest

from test_gpu_fused_multi import _launch

pytestmark = pytest.mark.gpu


def test_tensor_parallel_mlp_on_one_rank():
    _launch(1, 29881, "tp_worker.py", timeout=600)
    _launch(1, 29882, "tp_worker.py", "--rows", "512", "--hidden", "2048", "--ffn", "1024", timeout=600)


def test_tensor_parallel_mlp_fp8_on_one_rank():
    """Both fused kernels on block-scaled e4m3 operands against the PyTorch statement of the same arithmetic."""
    _launch(1, 29885, "tp_worker.py", "--fp8", timeout=600)
    _launch(1, 29886, "tp_worker.py", "--fp8", "--rows", "512", "--hidden", "2048", "--ffn", "1024", timeout=600)


def test_tensor_parallel_layer_forward_and_backward_on_one_rank():
    """Forward and backward of the whole tensor-parallel layer, and of the MLP half at a second shape, against float64 autograd."""
    _launch(1, 29888, "tp_layer_worker.py", timeout=600)
    _launch(1, 29889, "tp_layer_worker.py", "--what", "mlp", "--rows", "512", "--hidden", "2048", "--ffn", "1024", timeout=600)


def test_expert_parallel_layer_on_one_rank():
    _launch(1, 29883, "ep_worker.py", "--experts-local", "32", timeout=600)


def test_expert_parallel_layer_backward_on_one_rank():
    _launch(1, 29880, "ep_worker.py", "--experts-local", "32", "--backward", timeout=600)


def test_expert_parallel_layer_with_fp8_experts_on_one_rank():
    """The first expert GEMM on the received e4m3 rows and block-quantised weights (no dequantisation pass)."""
    _launch(1, 29887, "ep_worker.py", "--experts-local", "32", "--fp8-experts", timeout=600)


def test_device_initiated_layer_on_one_pe():
    """put+signal to itself, the atomics on its own words, the barrier of one: the device API's code paths on one GPU."""
    _launch(1, 29884, "shmem_worker.py", timeout=600)
