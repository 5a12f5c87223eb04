"""Causal attention over a sequence sharded across ranks, two ways: ring attention (key/value blocks travel
around the ring, online soft-max) and the Ulysses re-shard (all-to-all from sequence shards to head shards and
back). Both are checked against attention over the gathered sequence.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/long_context_attention.py
    ... --nproc-per-node 8 examples/long_context_attention.py --device cuda --seq 65536
"""
import argparse
import math
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from rocm_systems_b200.parallel.cp import ring_attention, ulysses_attention  # noqa: E402


def full_attention(q, k, v):
    s = q.shape[2]
    w = (q.float() @ k.float().transpose(-1, -2)) / math.sqrt(q.shape[-1])
    w = w.masked_fill(~torch.ones(s, s, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    return (torch.softmax(w, -1) @ v.float()).to(q.dtype)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", choices=["cpu", "cuda"], default="cpu")
    ap.add_argument("--seq", type=int, default=256, help="whole sequence length")
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--dim", type=int, default=32)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if a.device == "cuda":
        from rocm_systems_b200.parallel import init_process_group

        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        init_process_group()
        dev = torch.device("cuda", torch.cuda.current_device())
    else:
        dist.init_process_group("gloo")
        dev = torch.device("cpu")
    s_local = a.seq // world
    g = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn(1, a.heads, a.seq, a.dim, generator=g) for _ in range(3))
    shard = slice(rank * s_local, (rank + 1) * s_local)
    ql, kl, vl = (t[:, :, shard].contiguous().to(dev).requires_grad_(True) for t in (q, k, v))
    verify = a.seq <= 8192  # the check materialises the whole score matrix
    want = full_attention(q.to(dev), k.to(dev), v.to(dev))[:, :, shard] if verify else None

    worst = 0.0
    for name, fn in (("ring", ring_attention), ("ulysses", ulysses_attention)):
        out = fn(ql, kl, vl, causal=True)
        out.sum().backward()  # the backward pass runs the same exchanges in reverse
        err = float((out.detach() - want).abs().max()) if verify else float("nan")
        worst = max(worst, err if verify else 0.0)
        if rank == 0:
            print(f"{name:8s} tokens per rank {s_local}, max |error| vs unsharded attention: {err:.2e}, grad norm {float(ql.grad.norm()):.4f}", flush=True)
        ql.grad = kl.grad = vl.grad = None
    flag = torch.tensor([worst], dtype=torch.float32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    ok = float(flag) < 1e-4
    if rank == 0:
        print("long_context_attention OK" if ok else "long_context_attention MISMATCH", flush=True)
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
