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
    print(json.dumps({"cta_pairs_on_device": int(ops._lib_ops().b200ops_gemm_pairs_on_device())}), flush=True)
    for sh in args.shapes.split(","):
        M, N, K = (int(v) for v in sh.split("x"))
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        ours_med, ours_min = time_ms(lambda: ops.gemm_bf16_tn(a, b, out=out, bn=args.bn), flush, args.iters)
        err = ops.gemm_take_error()
        fl = 2.0 * M * N * K
        row = {"M": M, "N": N, "K": K, "ours_ms": ours_med, "ours_tflops": fl / ours_med / 1e9, "ours_best_tflops": fl / ours_min / 1e9, "gemm_error": err}
        # the CTA-pair kernel in the three operand orders of a linear layer: forward (both K-major), input gradient
        # (B read as the transpose of a row-major matrix), weight gradient (both operands transposes)
        at = torch.randn(K, M, device="cuda").to(torch.bfloat16)
        bt = torch.randn(K, N, device="cuda").to(torch.bfloat16)
        for bn in (128, 256):          # both tile widths, to check the automatic choice (pair_tn below) against
            med, _ = time_ms(lambda: ops.gemm(a, b, out=out, bn=bn), flush, args.iters)
            row[f"pair_tn_bn{bn}_ms"] = med
        for name, fa, fb in (("pair_tn", a, b), ("pair_nn", a, bt.t()), ("pair_tt", at.t(), bt.t())):
            med, best = time_ms(lambda: ops.gemm(fa, fb, out=out, bn=args.bn), flush, args.iters)
            row[name + "_ms"], row[name + "_tflops"] = med, fl / med / 1e9
            row[name + "_error"] = ops.gemm_take_error()
        if not args.only_ours:
            ref = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            lib_med, lib_min = time_ms(lambda: torch.matmul(a, b.t(), out=ref), flush, args.iters)
            ops.gemm_bf16_tn(a, b, out=out, bn=args.bn)
            row.update({"cublas_ms": lib_med, "cublas_tflops": fl / lib_med / 1e9, "ratio": lib_med / ours_med, "pair_tn_ratio": lib_med / row["pair_tn_ms"],
                        "max_abs_diff": float((out.float() - ref.float()).abs().max())})
            nn_med, _ = time_ms(lambda: torch.matmul(a, bt, out=ref), flush, args.iters)
            tt_med, _ = time_ms(lambda: torch.matmul(at.t(), bt, out=ref), flush, args.iters)
            row.update({"cublas_nn_ms": nn_med, "pair_nn_ratio": nn_med / row["pair_nn_ms"], "cublas_tt_ms": tt_med, "pair_tt_ratio": tt_med / row["pair_tt_ms"]})
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
