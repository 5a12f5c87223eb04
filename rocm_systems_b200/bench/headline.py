"""The headline figures of the collective stack in a form short enough to ride along with the training benchmark:

* ``collectives_vs_nccl``  per collective, stock-NCCL time / this library's time over a doubling-by-four ladder of
  message sizes (bf16, out of place, device-timed, max over ranks), as the minimum and the geometric mean of the ratio,
  plus the bus bandwidth of both at the largest size. The rccl-tests harness reports algbw / busbw per size and gates a
  run on the average busbw (rccl-tests/src/common.cpp:848-850, 1963-1986); this is the same measurement, summarised.
* ``tp_roofline``          the fused tensor-parallel MLP (all-gather -> GEMM + SwiGLU, GEMM -> reduce-scatter) at
  M = 8192 tokens, K = 8192, 28672 FFN columns split over the ranks: time against the slower of its FLOPs at the
  measured GEMM peak and its NVLink bytes at the measured link bandwidth.
* ``ep_roofline``          expert-parallel dispatch + combine (256 experts, top-8, hidden 7168, 4096 tokens per GPU)
  against its NVLink bytes at the measured link bandwidth, and the grouped expert GEMMs against the measured GEMM peak.

Every function is collective over the communicator: all ranks call it.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

LINK_GBS = 770.0            # measured peer-copy bandwidth per direction per GPU on this pool
FALLBACK_TFLOPS = 1590.0    # used when no measured-peaks file is present


def measured_bf16_tflops() -> tuple:
    """(TFLOP/s, "measured" | "fallback"): the burst cuBLAS bf16 figure written by the pool's driver, when present."""
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["bf16_tflops"]), "measured"
    except Exception:  # noqa: BLE001
        return FALLBACK_TFLOPS, "fallback"


def collectives_vs_nccl(comm, max_bytes: int = 256 << 20, min_bytes: int = 1 << 10, factor: int = 4, warmup: int = 5, iters: int = 20,
                        colls=("all_reduce", "reduce_scatter", "all_gather", "alltoall", "broadcast")) -> dict:
    """Needs an initialised ``torch.distributed`` NCCL process group next to ``comm``."""
    from .coll_sweep import sweep

    sizes = []
    s = min_bytes
    while s <= max_bytes:
        sizes.append(s)
        s *= factor
    send = torch.empty(max_bytes // 2, dtype=torch.bfloat16, device=comm.device).normal_()
    recv = torch.empty(max_bytes // 2, dtype=torch.bfloat16, device=comm.device)
    rows = sweep(comm, list(colls), sizes, torch.bfloat16, send, recv, warmup, iters, nccl=True)
    out = {"dtype": "bf16", "placement": "out of place", "sizes_bytes": sizes, "warmup": warmup, "iters": iters, "per_collective": {}}
    for c in colls:
        rs = [r for r in rows if r["coll"] == c]
        ratios = [r["nccl_us"] / r["ours_us"] for r in rs]
        worst = min(range(len(rs)), key=lambda i: ratios[i])
        out["per_collective"][c] = {
            "min_ratio_vs_nccl": min(ratios), "min_ratio_at_bytes": rs[worst]["bytes"],
            "geomean_ratio_vs_nccl": math.exp(sum(math.log(x) for x in ratios) / len(ratios)),
            "busbw_gbs_at_max": rs[-1]["ours_busbw"], "nccl_busbw_gbs_at_max": rs[-1]["nccl_busbw"],
            "ratios": [round(x, 3) for x in ratios],
        }
    return out


def tp_roofline(comm, total_rows: int = 8192, hidden: int = 8192, ffn_total: int = 28672, iters: int = 10) -> dict:
    from ..parallel.tp import TensorParallelMLP

    n = comm.nranks
    rows, f = total_rows // n, ffn_total // n
    mlp = TensorParallelMLP(comm, rows, hidden, f, comm.device, seed=11)
    g = torch.Generator(device=comm.device).manual_seed(comm.rank)
    mlp.my_rows().copy_(torch.randn(rows, hidden, device=comm.device, generator=g).to(torch.bfloat16))
    ms = _dev_ms(lambda: mlp.forward(None), comm, 3, iters)
    flops = 2.0 * total_rows * hidden * 2 * f + 2.0 * total_rows * f * hidden
    peak, kind = measured_bf16_tflops()
    t_compute = flops / (peak * 1e12) * 1e3
    link_bytes = (n - 1) / n * total_rows * hidden * 2          # gathered in, and the same amount of partial rows out
    t_link = link_bytes / (LINK_GBS * 1e9) * 1e3
    roof = max(t_compute, t_link)
    mlp.free()
    return {"shape": {"M": total_rows, "K": hidden, "ffn_per_rank": f, "tp": n}, "fused_ms": ms, "roofline_ms": roof, "compute_ms": t_compute,
            "link_ms_each_way": t_link, "fraction_of_roofline": roof / ms, "tflops_per_gpu": flops / (ms * 1e-3) / 1e12, "peak": f"{peak} TFLOP/s bf16 ({kind})"}


def ep_roofline(comm, experts_local: int = 32, hidden: int = 7168, ffn: int = 2048, topk: int = 8, tokens: int = 4096, iters: int = 5) -> dict:
    from ..parallel.ep import MoELayer

    n = comm.nranks
    moe = MoELayer(comm, experts_local, hidden, ffn, topk, tokens, seed=3)
    g = torch.Generator(device=comm.device).manual_seed(comm.rank)
    x = torch.randn(tokens, hidden, device=comm.device, generator=g).to(torch.bfloat16)
    logits = torch.randn(tokens, moe.E, device=comm.device, generator=g)
    moe.route(logits)

    def dc():
        moe.dispatch(x)
        moe.combine()

    dc_ms = _dev_ms(dc, comm, 2, iters)
    moe.dispatch(x)
    ex_ms = _dev_ms(moe.experts, comm, 2, iters)
    moe.combine()
    layer_ms = _dev_ms(lambda: moe.forward(x, logits), comm, 2, iters)
    remote = (n - 1) / n
    link_bytes = tokens * topk * (hidden + hidden // 128 * 4) * remote + tokens * topk * hidden * 2 * remote
    t_link = link_bytes / (LINK_GBS * 1e9) * 1e3
    peak, kind = measured_bf16_tflops()
    flops = 2.0 * tokens * topk * hidden * 3 * ffn              # rows per GPU on average = tokens * topk
    t_gemm = flops / (peak * 1e12) * 1e3
    moe.free()
    return {"shape": {"experts": moe.E, "topk": topk, "hidden": hidden, "ffn": ffn, "tokens_per_gpu": tokens, "ep": n},
            "dispatch_plus_combine_ms": dc_ms, "link_roofline_ms": t_link, "dispatch_combine_fraction_of_roofline": t_link / dc_ms,
            "experts_ms": ex_ms, "experts_fraction_of_peak": t_gemm / ex_ms, "layer_ms": layer_ms, "peak": f"{peak} TFLOP/s bf16 ({kind}), {LINK_GBS} GB/s link"}


def _dev_ms(fn, comm, warmup: int, iters: int) -> float:
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
