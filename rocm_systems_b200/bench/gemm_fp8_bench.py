"""Check and time the block-scaled fp8 GEMM and its quantisers against their PyTorch statements, next to the bf16
tcgen05 GEMM and the library bf16 GEMM on the same shapes. Between timed launches a buffer larger than the L2 is
rewritten.

    python -m rocm_systems_b200.bench.gemm_fp8_bench --check-shape 512x384x1024 --shapes 8192x8192x8192,8192x7168x8192

The check runs first, on the small shape, and the timing is skipped when it fails or when a bounded wait inside the
kernel ran out.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from ..ops import fp8
from ..ops import train_ops as ops
from .gemm_bench import time_ms


def check(M: int, N: int, K: int) -> dict:
    g = torch.Generator(device="cuda").manual_seed(3)
    x = (torch.randn(M, K, device="cuda", generator=g) * torch.logspace(-2, 1, M, device="cuda").unsqueeze(1)).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    xq, xs = fp8.quantize_act(x)
    wq, ws = fp8.quantize_weight(w)
    rxq, rxs = fp8.ref_quantize_act(x)
    rwq, rws = fp8.ref_quantize_weight(w)
    res = {
        "M": M, "N": N, "K": K,
        "act_scale_ok": bool(torch.allclose(xs, rxs, rtol=1e-6, atol=0)),
        "act_q_mismatch": int((xq.view(torch.uint8) != rxq.view(torch.uint8)).sum()),
        "w_scale_ok": bool(torch.allclose(ws, rws, rtol=1e-6, atol=0)),
        "w_q_mismatch": int((wq.view(torch.uint8) != rwq.view(torch.uint8)).sum()),
    }
    # The GEMM is checked on the oracle's quantised operands, so a quantiser difference cannot hide in it.
    got = fp8.gemm(rxq, rxs, rwq, rws).float()
    torch.cuda.synchronize()
    want = fp8.ref_gemm(rxq, rxs, rwq, rws).float()
    res["gemm_error_code"] = ops.gemm_take_error()
    res["gemm_max_abs_diff"] = float((got - want).abs().max())
    res["gemm_scale"] = float(want.abs().max())
    # one bf16 ulp of the largest value, plus fp32 summation-order noise
    res["gemm_ok"] = bool(res["gemm_error_code"] == 0 and res["gemm_max_abs_diff"] <= res["gemm_scale"] * 2 ** -7 + 1e-6)
    # the quantisers divide by the scale in IEEE arithmetic like the oracle does, so the codes agree exactly
    res["ok"] = bool(res["gemm_ok"] and res["act_scale_ok"] and res["w_scale_ok"] and res["act_q_mismatch"] == 0 and res["w_q_mismatch"] == 0)
    return res


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--check-shape", default="512x384x1024", help="MxNxK of the correctness run (N may be ragged, K a multiple of 128)")
    ap.add_argument("--shapes", default="4096x4096x4096,8192x8192x8192,8192x7168x8192,8192x8192x3584")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    M, N, K = (int(v) for v in args.check_shape.split("x"))
    rows = [check(M, N, K), check(300, 200, 256)]
    for r in rows:
        print(json.dumps(r), flush=True)
    if not all(r["ok"] for r in rows):
        print("fp8 GEMM check FAILED; not timing", flush=True)
        return 1
    flush = torch.zeros(192 << 20, dtype=torch.uint8, device="cuda")
    for sh in args.shapes.split(","):
        M, N, K = (int(v) for v in sh.split("x"))
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        aq, as_ = fp8.quantize_act(a)
        bq, bs = fp8.quantize_weight(b)
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        fl = 2.0 * M * N * K
        f8_med, f8_min = time_ms(lambda: fp8.gemm(aq, as_, bq, bs, out=out), flush, args.iters)
        code = ops.gemm_take_error()
        q_med, _ = time_ms(lambda: fp8.quantize_act(a), flush, args.iters)
        bf_med, _ = time_ms(lambda: ops.gemm_bf16_tn(a, b, out=out), flush, args.iters)
        lib_med, _ = time_ms(lambda: torch.matmul(a, b.t(), out=out), flush, args.iters)
        row = {"M": M, "N": N, "K": K, "fp8_ms": f8_med, "fp8_tflops": fl / f8_med / 1e9, "fp8_best_tflops": fl / f8_min / 1e9, "quant_act_ms": q_med,
               "bf16_tcgen05_ms": bf_med, "cublas_bf16_ms": lib_med, "fp8_vs_cublas_bf16": lib_med / f8_med, "gemm_error": code}
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
