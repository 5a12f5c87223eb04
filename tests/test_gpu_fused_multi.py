"""Multi-GPU tests of the fused compute+collective kernels, the device-initiated (shmem) layer and
the FSDP engine. Each test launches child ranks, one per GPU; a worker exits non-zero on any
mismatch against its unfused / single-rank oracle."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

from conftest import gpu_count

ROOT = Path(__file__).resolve().parent.parent
pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _launch(nproc: int, port: int, worker: str, *args: str, timeout: int = 900, extra_env=None) -> None:
    if gpu_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    env = dict(os.environ, **(extra_env or {}))
    env.setdefault("B200COLL_WAIT_TIMEOUT_MS", "5000")
    env.setdefault("B200COLL_BOOTSTRAP_TIMEOUT_MS", "60000")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(ROOT / "tests" / "workers" / worker), *args]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    sys.stdout.write(p.stdout[-4000:])
    sys.stderr.write(p.stderr[-4000:])
    assert p.returncode == 0


@pytest.mark.parametrize("nproc", [2, 8])
def test_tp_fused_mlp_matches_unfused(nproc):
    _launch(nproc, 29810 + nproc, "tp_worker.py")
    _launch(nproc, 29820 + nproc, "tp_worker.py", "--rows", "512", "--hidden", "2048", "--ffn", "1024")


@pytest.mark.parametrize("nproc", [2, 8])
def test_tp_fused_mlp_with_copy_engine_all_gather(nproc):
    """The all-gather side pulled by copy engines on a side stream (flags by stream memory writes), every SM on the GEMM."""
    _launch(nproc, 29970 + nproc, "tp_worker.py", "--comm-ctas", "-1")
    _launch(nproc, 29980 + nproc, "tp_worker.py", "--comm-ctas", "-1", "--rows", "512", "--hidden", "2048", "--ffn", "1024")


@pytest.mark.parametrize("nproc", [2, 8])
def test_tp_fused_mlp_fp8_matches_oracle(nproc):
    _launch(nproc, 29870 + nproc, "tp_worker.py", "--fp8")
    _launch(nproc, 29890 + nproc, "tp_worker.py", "--fp8", "--rows", "512", "--hidden", "2048", "--ffn", "1024")


@pytest.mark.parametrize("nproc", [2, 8])
def test_tp_layer_forward_and_backward_match_float64_autograd(nproc):
    """A whole tensor-parallel layer (attention and MLP halves, four fused kernels each way) and the MLP half alone at a
    second shape: outputs, input gradients, every weight shard's gradient and the norm-weight gradients."""
    _launch(nproc, 29740 + nproc, "tp_layer_worker.py", "--hidden", "2048", "--heads", "16", "--kv-heads", "8", "--ffn", "2048")
    _launch(nproc, 29750 + nproc, "tp_layer_worker.py", "--what", "mlp", "--rows", "512", "--hidden", "1024", "--ffn", "4096", "--comm-ctas", "-1")


@pytest.mark.parametrize("nproc", [2, 8])
def test_ep_dispatch_experts_combine(nproc):
    _launch(nproc, 29830 + nproc, "ep_worker.py")


@pytest.mark.parametrize("nproc", [2, 8])
def test_ep_backward_matches_float64_autograd(nproc):
    """Token, router-logit and expert-weight gradients of the layer (gate-gradient kernel, gradient gather, grouped GEMMs on
    transposed weights, unit-weight combine) against autograd of the unsharded layer."""
    _launch(nproc, 29760 + nproc, "ep_worker.py", "--backward")


@pytest.mark.parametrize("nproc", [2, 8])
def test_ep_with_fp8_experts(nproc):
    _launch(nproc, 29930 + nproc, "ep_worker.py", "--fp8-experts")


@pytest.mark.parametrize("nproc", [2, 8])
def test_shmem_put_get_signal_atomics(nproc):
    _launch(nproc, 29840 + nproc, "shmem_worker.py")


@pytest.mark.parametrize("nproc", [2, 8])
def test_shmem_device_collectives(nproc):
    _launch(nproc, 29950 + nproc, "shmem_worker.py", "--collectives")


@pytest.mark.parametrize("nproc", [2, 8])
def test_fsdp_matches_single_rank(nproc):
    """Shards and gradient buffers in symmetric memory (the default): parameter all-gather by the copy engines, zero-copy
    reduce-scatter+cast kernel."""
    _launch(nproc, 29850 + nproc, "fsdp_worker.py")


@pytest.mark.parametrize("nproc", [2, 8])
def test_fsdp_with_all_gather_kernel_matches_single_rank(nproc):
    """The parameter all-gather by the zero-copy all-gather kernel instead of the copy engines."""
    _launch(nproc, 29770 + nproc, "fsdp_worker.py", extra_env={"FSDP_COPY_ENGINE_GATHER": "0"})


@pytest.mark.parametrize("nproc", [2, 8])
def test_fsdp_with_staged_collectives_matches_single_rank(nproc):
    """Ordinary memory: the staged all-gather and the staged reduce-scatter+cast kernel; then with global-norm clipping."""
    _launch(nproc, 29860 + nproc, "fsdp_worker.py", extra_env={"FSDP_SYM_SHARDS": "0"})
    _launch(nproc, 29960 + nproc, "fsdp_worker.py", extra_env={"FSDP_CLIP": "1"})
