"""One small, self-contained run per kernel family on ONE GPU, in process: what a profiler is pointed at.

    python -m rocm_systems_b200.bench.kernel_cases --case gemm
    ncu --set full --clock-control none -k regex:gemmPairKernel -c 2 -o prof python -m rocm_systems_b200.bench.kernel_cases --case gemm

Cases (inputs are larger than the 126 MB L2 where the kernel streams memory, and at most a few GB in total):

    gemm        the CTA-pair tcgen05 GEMM in its three operand orders and the one-CTA kernel, 4096 x 4096 x 4096
    fp8         block-scaled e4m3 GEMM and its two quantisers, 4096 x 4096 x 4096
    tp          fused all-gather->GEMM(+SwiGLU) and GEMM->reduce-scatter on a communicator of one rank (tiles, policies,
                epilogues, staging and reducer run as on many ranks; nothing crosses a link)
    ep          expert-parallel route / dispatch / grouped expert GEMMs / combine on one rank (32 experts)
    train       RMSNorm forward + backward, RoPE, SwiGLU forward + backward, cross-entropy, embedding, AdamW at the shapes
                of the 8B model's step
    emu         the collective kernels' multi-rank paths (flag-in-data all-reduce, pipelined staged reduce with bulk loads,
                staged copy, FIFO send/recv, fused reduce-scatter+cast) as 4 emulated ranks in one cooperative kernel;
                must be started with B200COLL_EMULATE_RANKS=1 B200COLL_NVLS_ENABLE=0 in the environment

Every case prints one JSON line with CUDA-event times of what it ran, so the same command serves as the plain run that
precedes a capture.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os

import torch


def _time(fn, iters: int) -> float:
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def case_gemm(iters: int) -> dict:
    from ..ops import train_ops as ops

    M = N = K = 4096
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    at = torch.randn(K, M, device="cuda").to(torch.bfloat16)
    bt = torch.randn(K, N, device="cuda").to(torch.bfloat16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    res = {"shape": [M, N, K]}
    res["pair_tn_ms"] = _time(lambda: ops.gemm(a, b, out=out), iters)
    res["pair_nn_ms"] = _time(lambda: ops.gemm(a, bt.t(), out=out), iters)
    res["pair_tt_ms"] = _time(lambda: ops.gemm(at.t(), bt.t(), out=out), iters)
    res["one_cta_tn_ms"] = _time(lambda: ops.gemm_bf16_tn(a, b, out=out), iters)
    res["gemm_error"] = ops.gemm_take_error()
    return res


def case_fp8(iters: int) -> dict:
    from ..ops import fp8
    from ..ops import train_ops as ops

    M = N = K = 4096
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    res = {"shape": [M, N, K]}
    res["quant_act_ms"] = _time(lambda: fp8.quantize_act(x), iters)
    res["quant_weight_ms"] = _time(lambda: fp8.quantize_weight(w), iters)
    xq, xs = fp8.quantize_act(x)
    wq, ws = fp8.quantize_weight(w)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    res["gemm_fp8_ms"] = _time(lambda: fp8.gemm(xq, xs, wq, ws, out=out), iters)
    res["gemm_error"] = ops.gemm_take_error()
    return res


def _solo_comm():
    from ..comm import Communicator, get_unique_id

    torch.cuda.set_device(0)
    return Communicator(0, 1, get_unique_id(), 0)


def case_tp(iters: int) -> dict:
    from ..ops import train_ops as ops
    from ..parallel.tp import TensorParallelMLP, TensorParallelMLPFp8

    comm = _solo_comm()
    res = {}
    for name, cls in (("bf16", TensorParallelMLP), ("fp8", TensorParallelMLPFp8)):
        mlp = cls(comm, 4096, 4096, 3584, comm.device, seed=11)
        x = torch.randn(4096, 4096, device="cuda").to(torch.bfloat16)
        if name == "fp8":
            mlp.set_rows(x)
        else:
            mlp.my_rows().copy_(x)
        res[name + "_ag_gemm_ms"] = _time(mlp.ag_gemm, iters)
        res[name + "_gemm_rs_ms"] = _time(mlp.gemm_rs, iters)
        mlp.free()
    res["gemm_error"] = ops.gemm_take_error()
    comm.destroy()
    return res


def case_ep(iters: int) -> dict:
    from ..ops import train_ops as ops
    from ..parallel.ep import MoELayer

    comm = _solo_comm()
    res = {}
    for name, fp8e in (("bf16", False), ("fp8_experts", True)):
        moe = MoELayer(comm, 32, 4096, 1024, 8, 4096, seed=3, fp8_experts=fp8e)
        x = torch.randn(4096, 4096, device="cuda").to(torch.bfloat16)
        logits = torch.randn(4096, moe.E, device="cuda")
        res[name + "_layer_ms"] = _time(lambda: moe.forward(x, logits), iters)
        moe.free()
    res["gemm_error"] = ops.gemm_take_error()
    comm.destroy()
    return res


def case_train(iters: int) -> dict:
    from ..ops import train_ops as ops

    T, H, Fd, V = 4096, 4096, 14336, 128256
    res = {}
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16).requires_grad_(True)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    dy = torch.randn(T, H, device="cuda").to(torch.bfloat16)

    def norm():
        x.grad = w.grad = None
        ops.rmsnorm(x, w, 1e-5).backward(dy)

    res["rmsnorm_fwd_bwd_ms"] = _time(norm, iters)
    qkv = torch.randn(T, 48, 128, device="cuda").to(torch.bfloat16)
    table = ops.rope_table(4096, 128, 500000.0, "cuda")
    res["rope_ms"] = _time(lambda: ops.rope_(qkv, table, 40), iters)
    gu = torch.randn(T, 2 * Fd, device="cuda").to(torch.bfloat16).requires_grad_(True)
    da = torch.randn(T, Fd, device="cuda").to(torch.bfloat16)

    def swi():
        gu.grad = None
        ops.swiglu(gu).backward(da)

    res["swiglu_fwd_bwd_ms"] = _time(swi, iters)
    logits = torch.randn(T, V, device="cuda").to(torch.bfloat16)
    tgt = torch.randint(0, V, (T,), device="cuda")
    res["cross_entropy_ms"] = _time(lambda: ops.cross_entropy_inplace(logits, tgt, 1.0 / T), iters)
    table_w = torch.randn(V, H, device="cuda").to(torch.bfloat16)
    res["embedding_ms"] = _time(lambda: ops.embedding(tgt, table_w), iters)
    n = 218_112_000          # one layer of the 8B model
    master = torch.randn(n, device="cuda")
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    g = torch.randn(n, device="cuda").to(torch.bfloat16)
    p = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    res["adamw_ms"] = _time(lambda: ops.adamw_(master, m, v, g, p, 3e-4, (0.9, 0.95), 1e-8, 0.1, 1), iters)
    res["adamw_gbs"] = n * 30 / res["adamw_ms"] / 1e6
    return res


def case_emu(iters: int) -> dict:
    if os.environ.get("B200COLL_EMULATE_RANKS") != "1":
        raise SystemExit("the emu case needs B200COLL_EMULATE_RANKS=1 B200COLL_NVLS_ENABLE=0 in the environment")
    from .. import _lib

    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    lib = _lib.load()
    lib.b200collEmuSelftest.argtypes = [ctypes.c_int, ctypes.c_size_t, ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_int)]
    res = {}
    for nranks, count in ((4, (8 << 20) + 8),):
        wrong, status = ctypes.c_longlong(-1), ctypes.c_int(-1)
        rc = lib.b200collEmuSelftest(nranks, count, ctypes.byref(wrong), ctypes.byref(status))
        res[f"ranks{nranks}_count{count}"] = {"rc": rc, "wrong": wrong.value, "status": status.value}
    return res


CASES = {"gemm": case_gemm, "fp8": case_fp8, "tp": case_tp, "ep": case_ep, "train": case_train, "emu": case_emu}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=sorted(CASES))
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    res = CASES[a.case](a.iters)
    print(json.dumps({"case": a.case, **res}), flush=True)
    bad = res.get("gemm_error", 0) or any(isinstance(v, dict) and (v.get("rc") or v.get("wrong") or v.get("status")) for v in res.values())
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
