"""Copy-engine bandwidth grid: host-to-device, device-to-host, device-to-device and peer-to-peer
copies from 1 KiB to 512 MiB (20 sizes), mean and peak GB/s per size.

The counterpart of the reference runtime's async-copy performance suite
(rocr-runtime/rocrtst/suites/performance/memory_async_copy.cc: the same size grid, H2D / D2H / P2P,
mean and peak). One process drives all visible GPUs; copies are ``cudaMemcpyAsync`` through torch
on pinned host memory, timed with CUDA events on the copying stream after warm-up.

    python -m rocm_systems_b200.bench.copy_sweep [--peers] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

SIZES = [1 << k for k in range(10, 30)]  # 1 KiB .. 512 MiB


def _bw(dst: torch.Tensor, src: torch.Tensor, iters: int):
    # torch runs a copy between two GPUs on the source device's current stream; a host copy runs on the GPU side's stream
    stream = torch.cuda.current_stream(src.device if src.is_cuda else dst.device)
    for _ in range(2):
        dst.copy_(src, non_blocking=True)
    stream.synchronize()
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        dst.copy_(src, non_blocking=True)
        b.record(stream)
        stream.synchronize()
        times.append(a.elapsed_time(b) * 1e-3)
    n = src.numel()
    return n / (sum(times) / len(times)) / 1e9, n / min(times) / 1e9


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--peers", action="store_true", help="also copy to every other visible GPU")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--max", type=int, default=SIZES[-1])
    ap.add_argument("--json", default="")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("copy_sweep: no CUDA device", file=sys.stderr)
        return 1
    dev = torch.device("cuda", a.device)
    torch.cuda.set_device(dev)
    top = max(s for s in SIZES if s <= a.max)
    host = torch.empty(top, dtype=torch.uint8).pin_memory()
    d0 = torch.empty(top, dtype=torch.uint8, device=dev)
    d1 = torch.empty(top, dtype=torch.uint8, device=dev)
    peers = []
    if a.peers:
        for p in range(torch.cuda.device_count()):
            if p != a.device and torch.cuda.can_device_access_peer(a.device, p):
                peers.append((p, torch.empty(top, dtype=torch.uint8, device=torch.device("cuda", p))))
    cols = ["H2D", "D2H", "D2D"] + [f"P2P->{p}" for p, _ in peers]
    print(f"{'size':>12}  " + "  ".join(f"{c + ' mean/peak':>22}" for c in cols))
    rows = []
    for s in [x for x in SIZES if x <= top]:
        r = {"bytes": s, "H2D": _bw(d0[:s], host[:s], a.iters), "D2H": _bw(host[:s], d0[:s], a.iters), "D2D": _bw(d1[:s], d0[:s], a.iters)}
        for p, buf in peers:
            r[f"P2P->{p}"] = _bw(buf[:s], d0[:s], a.iters)
        rows.append(r)
        print(f"{s:>12}  " + "  ".join(f"{r[c][0]:>10.2f}/{r[c][1]:<11.2f}" for c in cols))
    if a.json:
        with open(a.json, "w") as f:
            json.dump(rows, f)
    return 0


if __name__ == "__main__":
    sys.exit(main())
