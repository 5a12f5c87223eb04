"""One rank of the fused tensor-parallel MLP check (all-gather->GEMM+SwiGLU, GEMM->reduce-scatter)
against the unfused composition, plus device timings of both."""
import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402

from rocm_systems_b200.comm import init_from_env  # noqa: E402
from rocm_systems_b200.ops import train_ops  # noqa: E402
from rocm_systems_b200.parallel.tp import TensorParallelMLP, TensorParallelMLPFp8  # noqa: E402


def timed(fn, comm, warmup=3, iters=10):
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=256)      # rows per rank
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--ffn", type=int, default=512)       # per rank
    ap.add_argument("--fp8", action="store_true")         # the block-scaled e4m3 form of both kernels
    ap.add_argument("--comm-ctas", type=int, default=0)   # CTAs that pull the peers' rows inside the all-gather kernel; -1: copy engines pull, no SM does
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    comm = init_from_env()
    rank, n = comm.rank, comm.nranks
    dev = comm.device
    mlp = (TensorParallelMLPFp8 if args.fp8 else TensorParallelMLP)(comm, args.rows, args.hidden, args.ffn, dev, seed=11, comm_ctas=args.comm_ctas)
    bad = []
    for trial in range(3):
        g = torch.Generator(device=dev).manual_seed(100 * trial + rank)
        x = torch.randn(args.rows, args.hidden, device=dev, generator=g).to(torch.bfloat16)
        ref = mlp.reference_forward(x).float()
        got = mlp.forward(x).float()
        torch.cuda.synchronize()
        code = train_ops.gemm_take_error()
        if code:
            bad.append(("gemm_error", code))
        err = (got - ref).abs().max().item()
        scale = ref.abs().max().item()
        if not (err <= 3e-2 * scale + 1e-3):
            bad.append(("mismatch", trial, err, scale))
    res = {"nranks": n, "rows_per_rank": args.rows, "hidden": args.hidden, "ffn_local": args.ffn, "comm_ctas": args.comm_ctas}
    if args.time and not bad:
        g = torch.Generator(device=dev).manual_seed(rank)
        x = torch.randn(args.rows, args.hidden, device=dev, generator=g).to(torch.bfloat16)
        if args.fp8:
            mlp.set_rows(x)
        else:
            mlp.my_rows().copy_(x)
        res["fused_ms"] = timed(lambda: mlp.forward(None), comm)
        if not args.fp8:
            res["unfused_ms"] = timed(lambda: mlp.reference_forward(x), comm)
        res["ag_gemm_ms"] = timed(lambda: mlp.ag_gemm(), comm)
        res["gemm_rs_ms"] = timed(lambda: mlp.gemm_rs(), comm)
        # the same two GEMMs with no communication at all (library GEMM), as the compute floor
        xg = torch.randn(n * args.rows, args.hidden, device=dev).to(torch.bfloat16)
        w13 = torch.cat([mlp.w_gate, mlp.w_up])
        res["local_gemm1_ms"] = timed(lambda: torch.mm(xg, w13.t()), comm)
        res["local_gemm2_ms"] = timed(lambda: torch.mm(mlp.act, mlp.w2.t()), comm)
        res["fp8"] = bool(args.fp8)
        M = n * args.rows
        flops = 2.0 * M * args.hidden * 2 * args.ffn + 2.0 * M * args.ffn * args.hidden
        res["fused_tflops_per_gpu"] = flops / (res["fused_ms"] * 1e-3) / 1e12
        res["gemm_error"] = train_ops.gemm_take_error()
    err = comm.async_error()
    if err:
        bad.append(("async_error", err, comm.last_error()))
    flags = comm.host_all_gather(bytes([1 if bad else 0]))
    if bad:
        print(f"[rank {rank}] TP MISMATCH: {bad}", flush=True)
    elif rank == 0:
        print(f"tp_worker OK on {n} ranks: {json.dumps(res)}", flush=True)
        if args.out:
            Path(args.out).write_text(json.dumps(res))
    mlp.free()
    comm.destroy()
    sys.exit(1 if any(f[0] for f in flags) else 0)


if __name__ == "__main__":
    main()
