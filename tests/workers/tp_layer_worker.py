"""One rank of the tensor-parallel layer check, forward AND backward: ``TensorParallelLayer`` (attention half and MLP half,
each an all-gather->GEMM kernel and a GEMM->reduce-scatter kernel per direction) against a float64 autograd statement of
the unsharded layer. Every rank gathers all ranks' weight shards and all tokens, evaluates the whole layer and its
gradients in float64, and compares its own rows of y and dx, its own shards' weight gradients and the norm-weight gradients.
``--what mlp`` checks the MLP half alone (any shape the fused kernels accept)."""
import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

from rocm_systems_b200.comm import init_from_env  # noqa: E402
from rocm_systems_b200.ops import train_ops  # noqa: E402
from rocm_systems_b200.parallel.tp import TensorParallelLayer, TensorParallelMLP, deinterleave_gate_up  # noqa: E402

REF = torch.float64


def gather(comm, t: torch.Tensor) -> list:
    """All ranks' copies of ``t`` (same shape everywhere), as a list indexed by rank."""
    t = t.contiguous()
    out = torch.empty(comm.nranks * t.numel(), dtype=t.dtype, device=t.device)
    comm.all_gather(t.view(-1), out)
    torch.cuda.synchronize()
    return [out[r * t.numel():(r + 1) * t.numel()].view(t.shape) for r in range(comm.nranks)]


def leaf(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(REF).requires_grad_(True)


def norm(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def mlp_parts(n2, shards):
    return sum((F.silu(n2 @ s["wg"].t()) * (n2 @ s["wu"].t())) @ s["w2"].t() for s in shards)


def attn_parts(n1, shards, hq, hkv, d, seq, theta):
    M = n1.shape[0]
    B = M // seq
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=n1.device, dtype=REF) / d))
    ang = torch.outer(torch.arange(seq, device=n1.device, dtype=REF), inv)
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]

    def rope(x):
        a, b = x[..., : d // 2], x[..., d // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

    total = 0
    for s in shards:
        qkv = (n1 @ s["wqkv"].t()).view(B, seq, hq + 2 * hkv, d)
        q, k, v = rope(qkv[:, :, :hq]), rope(qkv[:, :, hq:hq + hkv]), qkv[:, :, hq + hkv:]
        rep = hq // hkv
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(rep, 1), v.transpose(1, 2).repeat_interleave(rep, 1),
                                           is_causal=True)
        total = total + a.transpose(1, 2).reshape(M, hq * d) @ s["wo"].t()
    return total


def close(name, got, ref, tol, bad):
    err = (got.to(REF) - ref).abs().max().item()
    scale = ref.abs().max().item()
    if not (err <= tol * scale + 1e-6):
        bad.append((name, err, scale))
    return err / max(scale, 1e-30)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="layer", choices=["layer", "mlp"])
    ap.add_argument("--rows", type=int, default=256)      # rows per rank
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--ffn", type=int, default=1024)      # whole layer (split over the ranks)
    ap.add_argument("--seq", type=int, default=256)
    ap.add_argument("--comm-ctas", type=int, default=0)
    ap.add_argument("--tol", type=float, default=4e-2)
    ap.add_argument("--time", action="store_true")        # device time of forward + backward after the check
    ap.add_argument("--skip-check", action="store_true")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    comm = init_from_env()
    rank, n, dev = comm.rank, comm.nranks, comm.device
    bad, rel = [], {}
    g = torch.Generator(device=dev).manual_seed(77 + rank)
    x = torch.randn(args.rows, args.hidden, device=dev, generator=g).to(torch.bfloat16)
    dy = torch.randn(args.rows, args.hidden, device=dev, generator=g).to(torch.bfloat16)
    xs, dys = gather(comm, x), gather(comm, dy)
    x_full = leaf(torch.cat(xs))
    dy_full = torch.cat(dys).to(REF)
    lo, hi = rank * args.rows, (rank + 1) * args.rows
    theta, eps = 500000.0, 1e-5

    if args.what == "mlp":
        mod = TensorParallelMLP(comm, args.rows, args.hidden, args.ffn // n, dev, seed=5, comm_ctas=args.comm_ctas)
        mlps = [mod]
    else:
        mod = TensorParallelLayer(comm, args.rows, args.hidden, args.heads, args.kv_heads, args.ffn, args.seq, dev, eps=eps, seed=5, comm_ctas=args.comm_ctas)
        g2 = torch.Generator(device=dev).manual_seed(3)   # same on every rank: the norm weights are replicated
        mod.norm1 = (1.0 + 0.1 * torch.randn(args.hidden, device=dev, generator=g2)).to(torch.bfloat16)
        mod.norm2 = (1.0 + 0.1 * torch.randn(args.hidden, device=dev, generator=g2)).to(torch.bfloat16)
        mlps = [mod.mlp]
    mlp = mlps[0]
    shards_mlp = [{"wg": leaf(a), "wu": leaf(b), "w2": leaf(c)} for a, b, c in zip(gather(comm, mlp.w_gate), gather(comm, mlp.w_up), gather(comm, mlp.w2))]

    for trial in range(0 if args.skip_check else 2):   # the second pass runs on the buffers and call counters the first one left
        for s in shards_mlp:
            for t in s.values():
                t.grad = None
        x_full.grad = None
        if args.what == "mlp":
            y_ref = mlp_parts(x_full, shards_mlp)
            y_ref.backward(dy_full)
            y = mod.forward(x).clone()
            dx = mod.backward(dy).clone()
        else:
            att = mod.attn
            if trial == 0:
                shards_att = [{"wqkv": leaf(a), "wo": leaf(b)} for a, b in zip(gather(comm, att.w_qkv), gather(comm, att.w_o))]
                n1w, n2w = leaf(mod.norm1), leaf(mod.norm2)
            for s in shards_att:
                for t in s.values():
                    t.grad = None
            n1w.grad = n2w.grad = None
            h = x_full + attn_parts(norm(x_full, n1w, eps), shards_att, att.hq, att.hkv, att.d, args.seq, theta)
            y_ref = h + mlp_parts(norm(h, n2w, eps), shards_mlp)
            y_ref.backward(dy_full)
            y = mod.forward(x).clone()
            dx = mod.backward(dy).clone()
        torch.cuda.synchronize()
        code = train_ops.gemm_take_error()
        if code:
            bad.append(("gemm_error", code))
        tag = f"t{trial}."
        rel[tag + "y"] = close("y", y, y_ref.detach()[lo:hi], args.tol, bad)
        rel[tag + "dx"] = close("dx", dx, x_full.grad[lo:hi], args.tol, bad)
        mine = shards_mlp[rank]
        dwg, dwu = deinterleave_gate_up(mlp.grads["w13"], mlp.tile)
        rel[tag + "dw_gate"] = close("dw_gate", dwg, mine["wg"].grad, args.tol, bad)
        rel[tag + "dw_up"] = close("dw_up", dwu, mine["wu"].grad, args.tol, bad)
        rel[tag + "dw2"] = close("dw2", mlp.grads["w2"], mine["w2"].grad, args.tol, bad)
        if args.what == "layer":
            rel[tag + "dw_qkv"] = close("dw_qkv", mod.attn.grads["w_qkv"], shards_att[rank]["wqkv"].grad, args.tol, bad)
            rel[tag + "dw_o"] = close("dw_o", mod.attn.grads["w_o"], shards_att[rank]["wo"].grad, args.tol, bad)
            rel[tag + "dnorm1"] = close("dnorm1", mod.grads["norm1"], n1w.grad, args.tol, bad)
            rel[tag + "dnorm2"] = close("dnorm2", mod.grads["norm2"], n2w.grad, args.tol, bad)
    if args.time and not bad:
        def dev_ms(fn, warmup=3, iters=10):
            for _ in range(warmup):
                fn()
            torch.cuda.synchronize()
            comm.host_barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                fn()
            b.record()
            torch.cuda.synchronize()
            parts = comm.host_all_gather(float(a.elapsed_time(b) / iters).hex().encode().ljust(32))
            return max(float.fromhex(p.decode().strip()) for p in parts)

        M, H = n * args.rows, args.hidden
        f = args.ffn // n
        gemm_flops = 2.0 * M * H * 3 * f                     # gate, up, down of this rank's shard
        if args.what == "layer":
            att = mod.attn
            gemm_flops += 2.0 * M * H * (att.w_qkv.shape[0] + att.hq * att.d)
        rel["forward_ms"] = dev_ms(lambda: mod.forward(x))
        rel["forward_backward_ms"] = dev_ms(lambda: (mod.forward(x), mod.backward(dy)))
        rel["gemm_tflops_per_gpu_fwd_bwd"] = 3.0 * gemm_flops / (rel["forward_backward_ms"] * 1e-3) / 1e12
        rel["shape"] = {"rows_per_rank": args.rows, "hidden": H, "ffn_per_rank": f, "tp": n, "what": args.what}
    err = comm.async_error()
    if err:
        bad.append(("async_error", err, comm.last_error()))
    flags = comm.host_all_gather(bytes([1 if bad else 0]))
    if bad:
        print(f"[rank {rank}] TP LAYER MISMATCH: {bad}", flush=True)
    elif rank == 0:
        print(f"tp_layer_worker OK ({args.what}) on {n} ranks: {json.dumps({k: (round(v, 5) if isinstance(v, float) else v) for k, v in rel.items()})}", flush=True)
        if args.out:
            Path(args.out).write_text(json.dumps(rel))
    mod.free()
    comm.destroy()
    sys.exit(1 if any(f[0] for f in flags) else 0)


if __name__ == "__main__":
    main()
