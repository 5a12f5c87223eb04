"""Pipeline, ring-attention and Ulysses building blocks on CPU ranks (gloo): results and gradients
must equal the single-process computation."""
import multiprocessing as mp
import os
import socket
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _spawn(fn, world, *args):
    ctx = mp.get_context("spawn")
    port = _free_port()
    q = ctx.Queue()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, q, args)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    bad = [r for r in res if r[1] is not None]
    assert not bad, bad
    return {r[0]: r[2] for r in res}


def _entry(fn, rank, world, port, q, args):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world)})
    import traceback

    import torch.distributed as dist

    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        out = globals()[fn](rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, None, out))
    except Exception:  # noqa: BLE001 - reported to the parent
        q.put((rank, traceback.format_exc(), None))


def _attn_ref(q, k, v, causal):
    import torch

    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal, enable_gqa=k.shape[1] != q.shape[1])


def _cp_worker(rank, world, kind, causal):
    import torch

    from rocm_systems_b200.parallel import cp

    torch.manual_seed(0)
    B, H, Hkv, S, D = 2, 4, 2 if kind == "ring" else 4, 8 * world, 16
    q = torch.randn(B, H, S, D, dtype=torch.float64, requires_grad=True)
    k = torch.randn(B, Hkv, S, D, dtype=torch.float64, requires_grad=True)
    v = torch.randn(B, Hkv, S, D, dtype=torch.float64, requires_grad=True)
    w = torch.randn(B, H, S, D, dtype=torch.float64)
    ref = _attn_ref(q, k, v, causal)
    (ref * w).sum().backward()
    sl = slice(rank * (S // world), (rank + 1) * (S // world))
    ql, kl, vl = (t.detach()[:, :, sl].clone().requires_grad_(True) for t in (q, k, v))
    fn = cp.ring_attention if kind == "ring" else cp.ulysses_attention
    out = fn(ql, kl, vl, None, causal)
    (out * w[:, :, sl]).sum().backward()
    err = (out - ref[:, :, sl]).abs().max().item()
    gerr = max((a.grad - b.grad[:, :, sl]).abs().max().item() for a, b in ((ql, q), (kl, k), (vl, v)))
    assert err < 1e-5 and gerr < 1e-5, (err, gerr)   # fp32 accumulation inside the ring kernel
    return err


@pytest.mark.parametrize("kind", ["ring", "ulysses"])
@pytest.mark.parametrize("causal", [True, False])
def test_context_parallel_attention_matches_full(kind, causal):
    _spawn("_cp_worker", 2, kind, causal)


def test_ring_attention_four_ranks():
    _spawn("_cp_worker", 4, "ring", True)


def _pp_worker(rank, world, schedule, micro):
    import torch

    from rocm_systems_b200.parallel.pp import PipelineStage

    torch.manual_seed(1)
    width, batch = 32, 4
    layers = [torch.nn.Sequential(torch.nn.Linear(width, width), torch.nn.Tanh()).double() for _ in range(world)]
    xs = [torch.randn(batch, width, dtype=torch.float64) for _ in range(micro)]
    ts = [torch.randn(batch, width, dtype=torch.float64) for _ in range(micro)]
    loss_fn = torch.nn.functional.mse_loss
    # single-process reference: mean over the micro-batches
    ref_losses = []
    for x, t in zip(xs, ts):
        h = x
        for l in layers:
            h = l(h)
        loss = loss_fn(h, t)
        ref_losses.append(loss.item())
        (loss / micro).backward()
    want = [p.grad.clone() for p in layers[rank].parameters()]
    for l in layers:
        l.zero_grad()
    stage = PipelineStage(layers[rank], act_shape=(batch, width), act_dtype=torch.float64)
    losses = stage.run(xs if rank == 0 else None, ts if rank == world - 1 else None, loss_fn, n_micro=micro, schedule=schedule)
    for p, w in zip(layers[rank].parameters(), want):
        assert torch.allclose(p.grad, w, rtol=1e-10, atol=1e-12), (p.grad - w).abs().max()
    if rank == world - 1:
        assert all(abs(a - b) < 1e-12 for a, b in zip(losses, ref_losses))
    return stage.peak_alive


@pytest.mark.parametrize("schedule", ["1f1b", "gpipe"])
def test_pipeline_matches_single_process(schedule):
    alive = _spawn("_pp_worker", 2, schedule, 6)
    if schedule == "1f1b":
        assert alive[0] == 2 and alive[1] == 1      # stages - stage activations at most
    else:
        assert alive[0] == 6


def test_pipeline_four_stages_1f1b():
    alive = _spawn("_pp_worker", 4, "1f1b", 8)
    assert [alive[r] for r in range(4)] == [4, 3, 2, 1]


def test_1f1b_order():
    from rocm_systems_b200.parallel.pp import schedule_1f1b

    assert schedule_1f1b(0, 2, 3) == [("F", 0), ("F", 1), ("B", 0), ("F", 2), ("B", 1), ("B", 2)]
    assert schedule_1f1b(1, 2, 3) == [("F", 0), ("B", 0), ("F", 1), ("B", 1), ("F", 2), ("B", 2)]
    for st in range(4):
        o = schedule_1f1b(st, 4, 2)   # fewer micro-batches than stages
        assert sorted(o) == sorted([("F", 0), ("F", 1), ("B", 0), ("B", 1)])
