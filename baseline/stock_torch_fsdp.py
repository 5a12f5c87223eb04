"""The comparison arm of ``bench.py --impl reference``: Llama-3-8B trained by stock PyTorch alone.

The reference project ships no collective library source that could be built for this GPU (its RCCL and rocSHMEM
components are placeholders in the snapshot and HIP-only upstream), so the arm that stands in for it is what its
own benchmark notes name as the fallback: stock NCCL + cuBLAS on the same box. This file is that arm. It uses
``torch.distributed.fsdp.fully_shard`` on the ``nccl`` backend, ``torch.nn`` modules, ``F.scaled_dot_product_attention``,
``F.rms_norm``, ``F.cross_entropy`` and ``torch.optim.AdamW(fused=True)``: nothing of this repository's package is
imported, none of its shared objects is mapped.

Same job as the other arm: Llama-3-8B shape (32 layers, hidden 4096, 32 heads / 8 KV heads, FFN 14336, vocabulary
128256, RoPE theta 500000), bf16 compute with fp32 master weights and AdamW (``MixedPrecisionPolicy(param_dtype=bf16,
reduce_dtype=fp32)`` over fp32 parameters), sequence 4096, micro-batch 1 per GPU, synthetic tokens, random-init
weights, and the same two timed regions (device-resident batches with the loss left on the device; pinned host batches
copied in and the loss read back every step).

On one GPU nothing is sharded, so parameters, gradients and both moments in fp32 take 128 GB before any activation; if
the first warm-up step runs out of memory the arm rebuilds itself with per-layer activation checkpointing and says so in
its JSON line (``"activation_checkpointing": true``).
"""
from __future__ import annotations

import gc
import json
import math
import os
import sys

REF_UNAVAILABLE = ("reference snapshot has no RCCL/rocSHMEM sources and no Python package (pip: 'neither setup.py nor pyproject.toml "
                   "found'); its collective code is HIP/AMD-only and cannot build for B200")

CFG = dict(vocab=128256, hidden=4096, layers=32, heads=32, kv_heads=8, ffn=14336, rope_theta=500000.0, eps=1e-5, seq_len=4096)
TINY = dict(vocab=1024, hidden=256, layers=2, heads=4, kv_heads=2, ffn=512, rope_theta=500000.0, eps=1e-5, seq_len=512)


def build_model(c: dict, checkpoint: bool):
    import torch
    import torch.nn as nn
    import torch.nn.functional as F
    from torch.utils.checkpoint import checkpoint as ckpt

    d = c["hidden"] // c["heads"]

    def rope_table(seq: int, device):
        inv = 1.0 / (c["rope_theta"] ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
        ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
        return torch.polar(torch.ones_like(ang), ang)          # [S, d/2] complex64

    def apply_rope(x, table):                                    # x [B, S, h, d]
        xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], d // 2, 2))
        return torch.view_as_real(xc * table[None, :, None, :]).flatten(3).to(x.dtype)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.n1 = nn.Parameter(torch.ones(c["hidden"]))
            self.n2 = nn.Parameter(torch.ones(c["hidden"]))
            self.qkv = nn.Linear(c["hidden"], (c["heads"] + 2 * c["kv_heads"]) * d, bias=False)
            self.o = nn.Linear(c["heads"] * d, c["hidden"], bias=False)
            self.gate_up = nn.Linear(c["hidden"], 2 * c["ffn"], bias=False)
            self.down = nn.Linear(c["ffn"], c["hidden"], bias=False)

        def forward(self, x, table):
            b, s, _ = x.shape
            h = F.rms_norm(x, (c["hidden"],), self.n1, c["eps"])
            q, k, v = self.qkv(h).split([c["heads"] * d, c["kv_heads"] * d, c["kv_heads"] * d], -1)
            q = apply_rope(q.view(b, s, c["heads"], d), table).transpose(1, 2)
            k = apply_rope(k.view(b, s, c["kv_heads"], d), table).transpose(1, 2)
            v = v.view(b, s, c["kv_heads"], d).transpose(1, 2)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=c["heads"] != c["kv_heads"])
            x = x + self.o(a.transpose(1, 2).reshape(b, s, c["heads"] * d))
            g, u = self.gate_up(F.rms_norm(x, (c["hidden"],), self.n2, c["eps"])).chunk(2, -1)
            return x + self.down(F.silu(g) * u)

    class Llama(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(c["vocab"], c["hidden"])
            self.blocks = nn.ModuleList(Block() for _ in range(c["layers"]))
            self.norm = nn.Parameter(torch.ones(c["hidden"]))
            self.head = nn.Linear(c["hidden"], c["vocab"], bias=False)
            self.table = None

        def forward(self, tokens):
            if self.table is None or self.table.shape[0] != tokens.shape[1]:
                self.table = rope_table(tokens.shape[1], tokens.device)
            x = self.embed(tokens)
            for blk in self.blocks:
                x = ckpt(blk, x, self.table, use_reentrant=False) if checkpoint else blk(x, self.table)
            return self.head(F.rms_norm(x, (c["hidden"],), self.norm, c["eps"]))

    m = Llama()
    for p in m.parameters():
        if p.dim() == 2:
            nn.init.normal_(p, std=0.02)
    return m


def flops_per_token(c: dict) -> float:
    d = c["hidden"] // c["heads"]
    gemm = c["layers"] * (c["hidden"] * (c["heads"] + 2 * c["kv_heads"]) * d + c["hidden"] * c["hidden"] + 3 * c["hidden"] * c["ffn"]) + c["vocab"] * c["hidden"]
    return 6.0 * gemm + c["layers"] * 6 * c["seq_len"] * c["hidden"]


def run(args, clock_sampler_cls) -> None:
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29517")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    c = dict(CFG if args.model == "llama3_8b" else TINY)
    if args.seq:
        c["seq_len"] = args.seq
    if getattr(args, "layers", 0):
        c["layers"] = args.layers
    S, B, nb = c["seq_len"], 1, 4
    g = torch.Generator().manual_seed(1234 + rank)
    host_tok = [torch.randint(0, c["vocab"], (B, S), generator=g, dtype=torch.int64).pin_memory() for _ in range(nb)]
    host_tgt = [torch.randint(0, c["vocab"], (B, S), generator=g, dtype=torch.int64).pin_memory() for _ in range(nb)]
    dev_tok = [t.to(dev) for t in host_tok]
    dev_tgt = [t.to(dev) for t in host_tgt]
    mesh = init_device_mesh("cuda", (world,))

    def make(checkpoint: bool):
        torch.manual_seed(0)
        with torch.device(dev):
            model = build_model(c, checkpoint)
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
        for blk in model.blocks:
            fully_shard(blk, mesh=mesh, mp_policy=mp)
        fully_shard(model, mesh=mesh, mp_policy=mp)
        opt = torch.optim.AdamW(model.parameters(), lr=getattr(args, "lr", 3e-4), betas=(0.9, 0.95), weight_decay=0.1, fused=True)
        return model, opt

    def step(model, opt, tok, tgt):
        logits = model(tok)
        loss = F.cross_entropy(logits.float().view(-1, c["vocab"]), tgt.reshape(-1))
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss.detach()

    use_ckpt = bool(args.reference_checkpointing)
    model, opt = make(use_ckpt)
    try:
        step(model, opt, dev_tok[0], dev_tgt[0])
        torch.cuda.synchronize()
        oom = 0
    except torch.OutOfMemoryError:
        oom = 1
    flag = torch.tensor([oom], device=dev)
    dist.all_reduce(flag)
    if int(flag.item()) and not use_ckpt:
        del model, opt
        gc.collect()
        torch.cuda.empty_cache()
        use_ckpt = True
        model, opt = make(True)
    if getattr(args, "loss_curve", 0):
        curve = [float(step(model, opt, dev_tok[i % nb], dev_tgt[i % nb]).item()) for i in range(args.loss_curve)]
        if rank == 0:
            print(json.dumps({"impl": "reference", "n_gpus": world, "lr": getattr(args, "lr", 3e-4), "layers": c["layers"], "activation_checkpointing": use_ckpt,
                              "loss_curve": [round(x, 4) for x in curve]}))
        dist.barrier()
        dist.destroy_process_group()
        return

    for i in range(args.warmup):
        step(model, opt, dev_tok[i % nb], dev_tgt[i % nb])

    def sync_all():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    sync_all()
    sampler = clock_sampler_cls(local)
    if rank == 0:
        sampler.start()

    def timed(fn) -> float:
        sync_all()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(args.steps):
            fn(i)
        b.record()
        sync_all()
        t = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms_dev = timed(lambda i: step(model, opt, dev_tok[i % nb], dev_tgt[i % nb]))
    losses = []
    tok_d, tgt_d = torch.empty_like(dev_tok[0]), torch.empty_like(dev_tgt[0])

    def e2e_step(i):
        tok_d.copy_(host_tok[i % nb], non_blocking=True)
        tgt_d.copy_(host_tgt[i % nb], non_blocking=True)
        losses.append(float(step(model, opt, tok_d, tgt_d).item()))

    ms_e2e = None if args.no_e2e else timed(e2e_step)
    clocks = sampler.stop() if rank == 0 else {}
    tokens_per_step = world * B * S
    out = {
        "impl": "reference", "baseline_kind": "stock_nccl_torch_fsdp", "reference_unavailable": REF_UNAVAILABLE,
        "metric": "llama3_8b_fsdp_train_tokens_per_sec", "value": tokens_per_step * args.steps / (ms_dev / 1e3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic tokens uniform over the vocabulary (seeded), random-init weights N(0,0.02)",
        "config": {"model": "llama3-8b" if args.model == "llama3_8b" else "tiny", "global_batch": world * B, "seq_len": S, "parallelism": f"fsdp{world}",
                   "optimizer": "adamw fp32 master (torch fused)", "layers": c["layers"], "hidden": c["hidden"], "activation_checkpointing": use_ckpt,
                   "stack": f"torch {torch.__version__} fully_shard, nccl {'.'.join(map(str, torch.cuda.nccl.version()))}, cuBLAS, SDPA",
                   "l2": "working set per step (GBs of weights and activations) is far larger than the 126 MB L2; no flush needed"},
        "clocks": clocks, "gpu_launches": 0,
        "model_tflops_per_gpu": flops_per_token(c) * B * S / (ms_dev / args.steps / 1e3) / 1e12,
        "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 2 ** 30,
    }
    if ms_e2e is not None:
        out["e2e"] = {"value": tokens_per_step * args.steps / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * S * 8, "d2h_bytes_per_step": 4,
                      "ms_per_step": ms_e2e / args.steps, "last_loss": losses[-1] if losses else None, "losses": [round(x, 4) for x in losses]}
        if losses and not all(math.isfinite(x) for x in losses):
            out["e2e"]["non_finite_loss"] = True
    if rank == 0:
        print(json.dumps(out), flush=True)
    sync_all()
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit("run through: python bench.py --impl reference")
