"""A plain PyTorch Llama-style decoder trained with ``torch.distributed.fsdp.fully_shard`` on a chosen collective backend: this
package's (``b200coll``) or stock ``nccl``, the same script for both, so the two tokens/s figures differ by the collective
library only. On CPU ranks (``--device cpu``, backend gloo) it runs a tiny model, which is how the script itself is tested.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/torch_fsdp_llama.py --backend b200coll
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/torch_fsdp_llama.py --backend nccl
    ... --model llama3-8b --seq 4096            # the flagship shape (needs 8 GPUs)
"""
import argparse
import math
import os
import sys
import time
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from rocm_systems_b200.models.llama import LlamaConfig  # noqa: E402


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(dim)), eps

    def forward(self, x):
        return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def rope(x, theta: float):
    b, h, s, d = x.shape
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = torch.outer(torch.arange(s, device=x.device, dtype=torch.float32), inv)
    cos, sin = ang.cos()[None, None], ang.sin()[None, None]
    x1, x2 = x.float()[..., : d // 2], x.float()[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)


class Block(nn.Module):
    def __init__(self, c: LlamaConfig):
        super().__init__()
        self.c = c
        d = c.head_dim
        self.n1, self.n2 = RMSNorm(c.hidden, c.eps), RMSNorm(c.hidden, c.eps)
        self.qkv = nn.Linear(c.hidden, (c.heads + 2 * c.kv_heads) * d, bias=False)
        self.o = nn.Linear(c.heads * d, c.hidden, bias=False)
        self.gate_up = nn.Linear(c.hidden, 2 * c.ffn, bias=False)
        self.down = nn.Linear(c.ffn, c.hidden, bias=False)

    def forward(self, x):
        c, d = self.c, self.c.head_dim
        b, s, _ = x.shape
        q, k, v = self.qkv(self.n1(x)).split([c.heads * d, c.kv_heads * d, c.kv_heads * d], -1)
        q = rope(q.view(b, s, c.heads, d).transpose(1, 2), c.rope_theta)
        k = rope(k.view(b, s, c.kv_heads, d).transpose(1, 2), c.rope_theta)
        v = v.view(b, s, c.kv_heads, d).transpose(1, 2)
        rep = c.heads // c.kv_heads
        a = F.scaled_dot_product_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1), is_causal=True)
        x = x + self.o(a.transpose(1, 2).reshape(b, s, c.heads * d))
        g, u = self.gate_up(self.n2(x)).chunk(2, -1)
        return x + self.down(F.silu(g) * u)


class Llama(nn.Module):
    def __init__(self, c: LlamaConfig):
        super().__init__()
        self.embed = nn.Embedding(c.vocab, c.hidden)
        self.blocks = nn.ModuleList(Block(c) for _ in range(c.layers))
        self.norm = RMSNorm(c.hidden, c.eps)
        self.head = nn.Linear(c.hidden, c.vocab, bias=False)

    def forward(self, tokens):
        x = self.embed(tokens)
        for blk in self.blocks:
            x = blk(x)
        return self.head(self.norm(x))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", choices=["b200coll", "nccl", "gloo"], default="b200coll")
    ap.add_argument("--device", choices=["cuda", "cpu"], default="cuda")
    ap.add_argument("--model", default="", help="a name LlamaConfig.by_name knows; default: tiny")
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--batch", type=int, default=1, help="sequences per rank and step")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    cfg = LlamaConfig.by_name(a.model) if a.model else LlamaConfig.tiny(64)
    if a.seq:
        cfg.seq_len = a.seq
    if a.device == "cpu":
        dist.init_process_group("gloo")
        dev, dtype = torch.device("cpu"), torch.float32
    else:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dev, dtype = torch.device("cuda", torch.cuda.current_device()), torch.bfloat16
        if a.backend == "b200coll":
            from rocm_systems_b200.parallel import init_process_group

            init_process_group()
        else:
            dist.init_process_group(a.backend)
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    torch.manual_seed(0)
    model = Llama(cfg).to(dev, dtype)
    mesh = init_device_mesh(dev.type, (world,))
    for blk in model.blocks:        # one gather / reduce-scatter unit per layer, then the embedding, norm and head together
        fully_shard(blk, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    g = torch.Generator().manual_seed(1 + rank)
    losses, t0 = [], 0.0
    for step in range(a.warmup + a.steps):
        if step == a.warmup:
            if dev.type == "cuda":
                torch.cuda.synchronize()
            dist.barrier()
            t0 = time.perf_counter()
        tok = torch.randint(0, cfg.vocab, (a.batch, cfg.seq_len + 1), generator=g).to(dev)
        logits = model(tok[:, :-1])
        loss = F.cross_entropy(logits.float().view(-1, cfg.vocab), tok[:, 1:].reshape(-1))
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        losses.append(float(loss.detach()))
    if dev.type == "cuda":
        torch.cuda.synchronize()
    dist.barrier()
    dt = time.perf_counter() - t0
    ok = all(math.isfinite(x) for x in losses)
    if rank == 0:
        tps = a.steps * a.batch * cfg.seq_len * world / dt
        print(f"torch FSDP on {dist.get_backend()} x{world}: {cfg.param_count() / 1e6:.1f} M parameters, seq {cfg.seq_len}, "
              f"{tps:,.0f} tokens/s, loss {losses[0]:.3f} -> {losses[-1]:.3f}", flush=True)
        print("torch_fsdp_llama OK" if ok else "torch_fsdp_llama: non-finite loss", flush=True)
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
