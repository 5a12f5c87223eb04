"""Measure this GPU's empirical ceilings: device-memory copy bandwidth, L2-resident copy bandwidth,
and dense bf16 / fp16 / tf32 / fp32 matrix-multiply rates (library GEMM, and this package's tcgen05
GEMM for bf16), each as a burst figure and as a sustained one. The result is the JSON the roofline
and counters tools read as ``--peaks``.

The counterpart of the reference's empirical roofline step (rocprofiler-compute runs prebuilt
micro-benchmarks per architecture, utils/rooflines/, and prints HBM / L2 / LDS bandwidth and peak
FLOP rates, docs/how-to/profile/mode.rst:139-159).

    python -m rocm_systems_b200.bench.empirical_roofline -o peaks.json

Timing: CUDA events, three warm-up calls, best of ``--repeat`` for the burst figure and a
``--sustain`` second loop for the sustained one; buffers larger than L2 for the HBM figure.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def _time(fn, repeat: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(repeat):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) * 1e-3)
    return best


def _sustained(fn, seconds: float) -> float:
    """Average time per call over a loop of about ``seconds`` (clocks settle under the power cap)."""
    torch.cuda.synchronize()
    t_call = _time(fn, 2)
    n = max(5, int(seconds / max(t_call, 1e-6)))
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e-3 / n


def measure(repeat: int = 10, sustain: float = 2.0, with_own_gemm: bool = True) -> dict:
    dev = torch.device("cuda", torch.cuda.current_device())
    props = torch.cuda.get_device_properties(dev)
    out = {"device": props.name, "sms": props.multi_processor_count, "measured_at": time.strftime("%Y-%m-%dT%H:%M:%S")}
    # device memory: 1 GiB -> 1 GiB copy, read + write bytes
    n = 1 << 30
    src, dst = torch.empty(n, dtype=torch.uint8, device=dev), torch.empty(n, dtype=torch.uint8, device=dev)
    out["hbm_gbs"] = 2 * n / _time(lambda: dst.copy_(src), repeat) / 1e9
    # L2-resident: 32 MiB -> 32 MiB, well inside the cache
    m = 32 << 20
    out["l2_gbs"] = 2 * m / _time(lambda: dst[:m].copy_(src[:m]), repeat) / 1e9
    del src, dst
    # matrix multiply
    size = 8192
    flops = 2.0 * size ** 3
    for name, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16), ("fp32", torch.float32)):
        a = torch.randn(size, size, device=dev, dtype=dt)
        b = torch.randn(size, size, device=dev, dtype=dt)
        if name == "fp32":
            torch.backends.cuda.matmul.allow_tf32 = True
            out["tf32_tflops"] = flops / _time(lambda: torch.mm(a, b), repeat) / 1e12
            torch.backends.cuda.matmul.allow_tf32 = False
        out[f"{name}_tflops"] = flops / _time(lambda: torch.mm(a, b), repeat) / 1e12
        if name == "bf16":
            out["bf16_tflops_sustained"] = flops / _sustained(lambda: torch.mm(a, b), sustain) / 1e12
            if with_own_gemm:
                try:
                    from ..ops import train_ops

                    c = torch.empty(size, size, device=dev, dtype=dt)
                    bt = b.t().contiguous()
                    out["bf16_tflops_tcgen05_kernel"] = flops / _time(lambda: train_ops.gemm_bf16_tn(a, bt, c), repeat) / 1e12
                except Exception as e:  # noqa: BLE001 - the ceilings are still valid without this row
                    out["bf16_tflops_tcgen05_kernel_error"] = str(e)
        del a, b
    out["ridge_flop_per_byte_bf16"] = out["bf16_tflops"] * 1e3 / out["hbm_gbs"]
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("-o", "--output", default="")
    ap.add_argument("--repeat", type=int, default=10)
    ap.add_argument("--sustain", type=float, default=2.0)
    ap.add_argument("--no-own-gemm", action="store_true")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("empirical_roofline: no CUDA device", file=sys.stderr)
        return 1
    res = measure(a.repeat, a.sustain, not a.no_own_gemm)
    text = json.dumps(res, indent=1)
    print(text)
    if a.output:
        with open(a.output, "w") as f:
            f.write(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
