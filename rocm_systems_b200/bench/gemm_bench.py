"""Device-timed comparison of the hand-written tcgen05 GEMM with the library GEMM (cuBLAS through
``torch.matmul``) on bf16 ``C = A @ B.T``. Between timed launches a buffer larger than the 126 MB
L2 is rewritten, so every launch starts cold.

    python -m rocm_systems_b200.bench.gemm_bench --shapes 8192x8192x8192,8192x7168x8192 --out gemm.json
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import train_ops as ops


def time_ms(fn, flush, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        flush.add_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="4096x4096x4096,8192x8192x8192,8192x7168x8192,8192x8192x3584,4096x6144x4096,4096x28672x4096")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--only-ours", action="store_true")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    flush = torch.zeros(192 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    for sh in args.shapes.split(","):
        M, N, K = (int(v) for v in sh.split("x"))
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        ours_med, ours_min = time_ms(lambda: ops.gemm_bf16_tn(a, b, out=out, bn=args.bn), flush, args.iters)
        err = ops.gemm_take_error()
        fl = 2.0 * M * N * K
        row = {"M": M, "N": N, "K": K, "ours_ms": ours_med, "ours_tflops": fl / ours_med / 1e9, "ours_best_tflops": fl / ours_min / 1e9, "gemm_error": err}
        if not args.only_ours:
            ref = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            lib_med, lib_min = time_ms(lambda: torch.matmul(a, b.t(), out=ref), flush, args.iters)
            row.update({"cublas_ms": lib_med, "cublas_tflops": fl / lib_med / 1e9, "ratio": lib_med / ours_med,
                        "max_abs_diff": float((out.float() - ref.float()).abs().max())})
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
