"""GPU tests of the collective library: single-GPU paths in-process, multi-GPU as child ranks."""
import os
import subprocess
import sys
import time
from pathlib import Path

import pytest
import torch

from conftest import gpu_count

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def solo_comm():
    from rocm_systems_b200.comm import Communicator, get_unique_id

    torch.cuda.set_device(0)
    c = Communicator(0, 1, get_unique_id(), 0)
    yield c
    torch.cuda.synchronize()
    c.destroy()


def test_single_rank_collectives(solo_comm):
    c = solo_comm
    x = torch.arange(1000, dtype=torch.float32, device="cuda")
    y = torch.zeros_like(x)
    c.all_reduce(x, y)
    c.all_gather(x, y)
    c.reduce_scatter(x, y)
    c.broadcast(x, y, root=0)
    torch.cuda.synchronize()
    assert torch.equal(x, y)
    # PreMulSum rescales even on one rank, so it runs the reduce kernel
    op = c.premul_sum(3.0, torch.float32)
    c.all_reduce(x, y, op=op)
    torch.cuda.synchronize()
    assert torch.equal(y, 3.0 * x)
    c.redop_destroy(op)
    # send to self pairs with receive from self
    z = torch.zeros_like(x)
    c.group_start()
    c.send(x, 0)
    c.recv(z, 0)
    c.group_end()
    torch.cuda.synchronize()
    assert torch.equal(x, z)
    assert c.async_error() == 0


def test_premul_sum_reads_a_device_scalar_in_stream_order(solo_comm):
    """The scalar is written by earlier work on the stream and changed right after the call: the kernel must see the value
    that stream order gives it, the enqueue must not wait for the stream, and the call must be capturable in a graph."""
    c = solo_comm
    x = torch.arange(4096, dtype=torch.float32, device="cuda")
    y = torch.zeros_like(x)
    scalar = torch.zeros(1, dtype=torch.float32, device="cuda")
    op = c.premul_sum_device(scalar)
    scalar.fill_(5.0)            # stream-ordered before the collective
    c.all_reduce(x, y, op=op)
    scalar.fill_(-1.0)           # stream-ordered after it
    torch.cuda.synchronize()
    assert torch.equal(y, 5.0 * x)
    # captured: the scalar of each replay is whatever the stream holds at that point
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        c.all_reduce(x, y, op=op)          # warm-up on the capture stream
        side.synchronize()
        with torch.cuda.graph(g, stream=side):
            c.all_reduce(x, y, op=op, stream=side)
    for v in (2.0, 7.0):
        scalar.fill_(v)
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, v * x)
    c.redop_destroy(op)
    assert c.async_error() == 0


def test_bounded_wait_reports_instead_of_hanging():
    """A wait on a flag nothing sets runs out of budget: the kernel returns, the status word is
    set, the communicator reports a remote error, and the CUDA context stays usable."""
    from rocm_systems_b200.comm import Communicator, get_unique_id

    torch.cuda.set_device(0)
    c = Communicator(0, 1, get_unique_id(), 0)
    t0 = time.time()
    c._test_wait_timeout(300)
    torch.cuda.synchronize()
    assert time.time() - t0 < 10
    deadline = time.time() + 5
    err = 0
    while time.time() < deadline and err == 0:
        err = c.async_error()
        time.sleep(0.02)
    assert err == 6, c.last_error()  # ncclRemoteError
    assert "timed out" in c.last_error()
    # the context is alive: ordinary work still runs
    a = torch.ones(1024, device="cuda")
    assert float(a.sum().item()) == 1024.0
    c.abort()


@pytest.mark.multigpu
@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_multi_gpu_sweep(nproc):
    if gpu_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    env = dict(os.environ)
    env.setdefault("B200COLL_WAIT_TIMEOUT_MS", "5000")
    env.setdefault("B200COLL_BOOTSTRAP_TIMEOUT_MS", "60000")
    port = 29600 + nproc
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(ROOT / "tests" / "workers" / "coll_worker.py"), "--quick"]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    sys.stdout.write(p.stdout[-4000:])
    sys.stderr.write(p.stderr[-4000:])
    assert p.returncode == 0


@pytest.mark.multigpu
@pytest.mark.parametrize("nproc", [2, 8])
def test_torch_distributed_backend(nproc):
    if gpu_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    env = dict(os.environ)
    env.setdefault("B200COLL_WAIT_TIMEOUT_MS", "5000")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(29700 + nproc), str(ROOT / "tests" / "workers" / "dist_worker.py")]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    sys.stdout.write(p.stdout[-4000:])
    sys.stderr.write(p.stderr[-4000:])
    assert p.returncode == 0


@pytest.mark.multigpu
def test_large_messages_through_many_pipeline_chunks():
    """80 MB messages (several pipeline chunks with a short last one) for every dtype and operator,
    bit-exact; once with the default chunking and once with 1 MiB chunks."""
    if gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    for i, extra in enumerate(({}, {"B200COLL_PIPELINE_CHUNK": "1M"})):
        env = dict(os.environ, **extra)
        env.setdefault("B200COLL_WAIT_TIMEOUT_MS", "5000")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
               "--master-port", str(29650 + i), str(ROOT / "tests" / "workers" / "coll_worker.py")]
        p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
        sys.stdout.write(p.stdout[-3000:])
        sys.stderr.write(p.stderr[-3000:])
        assert p.returncode == 0


@pytest.mark.multigpu
def test_mismatched_window_offsets_fall_back_to_staging():
    """Buffers in one symmetric window but at rank-dependent offsets: with the cross-rank check on, nobody takes the
    zero-copy path and the results stay exact."""
    if gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, B200COLL_CHECK_SYMMETRIC="1")
    env.setdefault("B200COLL_WAIT_TIMEOUT_MS", "5000")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29661", str(ROOT / "tests" / "workers" / "sym_offset_worker.py")]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    sys.stdout.write(p.stdout[-3000:])
    sys.stderr.write(p.stderr[-3000:])
    assert p.returncode == 0
