"""One rank of the expert-parallel MoE check: fused route/dispatch/experts/combine against the
plain PyTorch composition, plus device timings of the stages."""
import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402

from rocm_systems_b200.comm import init_from_env  # noqa: E402
from rocm_systems_b200.ops import train_ops  # noqa: E402
from rocm_systems_b200.parallel.ep import MoELayer, dequantize_e4m3_per128, quantize_e4m3_per128  # noqa: E402


def dev_ms(fn, comm, warmup=2, iters=5):
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
    ms = a.elapsed_time(b) / iters
    parts = comm.host_all_gather(float(ms).hex().encode().ljust(32))
    return max(float.fromhex(p.decode().strip()) for p in parts)


def gather(comm, t):
    """All ranks' copies of ``t`` (same shape everywhere) concatenated along the first axis."""
    t = t.contiguous()
    out = torch.empty(comm.nranks * t.numel(), dtype=t.dtype, device=t.device)
    comm.all_gather(t.view(-1), out)
    torch.cuda.synchronize()
    return out.view(comm.nranks * t.shape[0], *t.shape[1:])


def check_backward(moe, comm, x, logits, dy, tol, bad):
    """Forward + backward of the layer against float64 autograd of the whole (unsharded) layer over all ranks' tokens, the
    fp8 transport of the dispatched rows treated as the identity in the backward direction."""
    F = torch.nn.functional
    D = torch.float64
    T, k, el, rank = moe.T, moe.k, moe.el, comm.rank
    X, L, DY = gather(comm, x), gather(comm, logits), gather(comm, dy).to(D)
    WG, WU, WD = (gather(comm, w).to(D).requires_grad_(True) for w in (moe.w_gate, moe.w_up, moe.w_down))
    Xl = X.to(D).requires_grad_(True)
    Ll = L.to(D).requires_grad_(True)
    Xq = dequantize_e4m3_per128(*quantize_e4m3_per128(X)).to(D)
    Xe = Xl + (Xq - Xl).detach()
    top_v, top_i = torch.topk(Ll, k, dim=-1)
    w = torch.softmax(top_v, dim=-1)
    out = torch.zeros_like(Xl)
    for e in range(moe.E):
        t, r = (top_i == e).nonzero(as_tuple=True)
        if t.numel() == 0:
            continue
        rows = Xe[t]
        y = (F.silu(rows @ WG[e].t()) * (rows @ WU[e].t())) @ WD[e].t()
        out = out.index_add(0, t, w[t, r].unsqueeze(-1) * y)
    out.backward(DY)
    got = moe.forward(x, logits).clone()
    dx, dlogits = moe.backward(dy)
    torch.cuda.synchronize()
    dwg, dwu, dwd = moe.expert_weight_grads()
    lo, hi = rank * T, (rank + 1) * T
    e0, e1 = rank * el, (rank + 1) * el
    rel = {}
    for name, a, b in (("y", got, out.detach()[lo:hi]), ("dx", dx, Xl.grad[lo:hi]), ("dlogits", dlogits, Ll.grad[lo:hi]),
                       ("dw_gate", dwg, WG.grad[e0:e1]), ("dw_up", dwu, WU.grad[e0:e1]), ("dw_down", dwd, WD.grad[e0:e1])):
        err = (a.to(D) - b).abs().max().item()
        scale = b.abs().max().item()
        rel[name] = err / max(scale, 1e-30)
        if not (err <= tol * scale + 1e-7):
            bad.append(("backward", name, err, scale))
    return rel


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backward", action="store_true")      # also check the layer's gradients against float64 autograd
    ap.add_argument("--experts-local", type=int, default=16)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--ffn", type=int, default=256)
    ap.add_argument("--topk", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--fp8-experts", action="store_true")   # first expert GEMM on the received fp8 rows
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--skip-check", action="store_true")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    comm = init_from_env()
    rank, n = comm.rank, comm.nranks
    dev = comm.device
    moe = MoELayer(comm, args.experts_local, args.hidden, args.ffn, args.topk, args.tokens, seed=3, fp8_experts=args.fp8_experts)
    bad = []
    res = {"nranks": n, "experts": moe.E, "topk": args.topk, "hidden": args.hidden, "ffn": args.ffn, "tokens_per_rank": args.tokens, "cap": moe.cap}
    if not args.skip_check:
        for trial in range(3):  # three calls: both parities of the double-buffered counters get reused
            g = torch.Generator(device=dev).manual_seed(50 * trial + rank)
            x = torch.randn(args.tokens, args.hidden, device=dev, generator=g).to(torch.bfloat16)
            logits = torch.randn(args.tokens, moe.E, device=dev, generator=g)
            ref = moe.reference_forward(x, logits).float()
            got = moe.forward(x, logits).float()
            torch.cuda.synchronize()
            code = train_ops.gemm_take_error()
            if code:
                bad.append(("gemm_error", code))
            counts, dropped = moe.counts()
            if dropped:
                bad.append(("dropped", dropped))
            # routing must agree with torch.topk
            tv, ti = torch.topk(logits, args.topk, dim=-1)
            if not torch.equal(moe.top_idx.long(), ti):
                bad.append(("route_idx", int((moe.top_idx.long() != ti).sum())))
            if not torch.allclose(moe.top_w, torch.softmax(tv, -1), rtol=1e-4, atol=1e-6):
                bad.append(("route_w",))
            err = (got - ref).abs().max().item()
            scale = ref.abs().max().item()
            if not (err <= 3e-2 * scale + 1e-4):
                bad.append(("mismatch", trial, err, scale))
            res["rows_received"] = int(sum(counts))
        if args.backward and not bad:
            for trial in range(2):
                g = torch.Generator(device=dev).manual_seed(900 + 50 * trial + rank)
                x = torch.randn(args.tokens, args.hidden, device=dev, generator=g).to(torch.bfloat16)
                logits = torch.randn(args.tokens, moe.E, device=dev, generator=g)
                dy = torch.randn(args.tokens, args.hidden, device=dev, generator=g).to(torch.bfloat16)
                res[f"backward_rel_err_{trial}"] = {k: round(v, 5) for k, v in check_backward(moe, comm, x, logits, dy, 4e-2, bad).items()}
                code = train_ops.gemm_take_error()
                if code:
                    bad.append(("gemm_error", code))
    if args.time and not bad:
        g = torch.Generator(device=dev).manual_seed(rank)
        x = torch.randn(args.tokens, args.hidden, device=dev, generator=g).to(torch.bfloat16)
        logits = torch.randn(args.tokens, moe.E, device=dev, generator=g)
        moe.route(logits)

        def dispatch_combine_only():
            moe.dispatch(x)
            moe.combine()

        res["layer_ms"] = dev_ms(lambda: moe.forward(x, logits), comm)
        res["dispatch_plus_combine_ms"] = dev_ms(dispatch_combine_only, comm)
        res["dispatch_ms"] = None
        # dispatch alone cannot be looped without its combine (the barrier lives there), so derive it
        moe.dispatch(x)
        res["experts_ms"] = dev_ms(lambda: moe.experts(), comm)
        moe.combine()
        H, k, T = args.hidden, args.topk, args.tokens
        remote = (n - 1) / n
        res["dispatch_bytes_remote"] = T * k * (H + H // 128 * 4) * remote
        res["combine_bytes_remote"] = T * k * H * 2 * remote
        res["gemm_error"] = train_ops.gemm_take_error()
    err = comm.async_error()
    if err:
        bad.append(("async_error", err, comm.last_error()))
    flags = comm.host_all_gather(bytes([1 if bad else 0]))
    if bad:
        print(f"[rank {rank}] EP FAILURES: {bad}", flush=True)
    elif rank == 0:
        print(f"ep_worker OK on {n} ranks: {json.dumps(res)}", flush=True)
        if args.out:
            Path(args.out).write_text(json.dumps(res))
    moe.free()
    comm.destroy()
    sys.exit(1 if any(f[0] for f in flags) else 0)


if __name__ == "__main__":
    main()
