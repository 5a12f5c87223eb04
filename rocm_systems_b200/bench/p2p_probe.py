"""Peer-to-peer probe: bandwidth of remote stores (put) and remote loads (get) from this GPU to
every peer, and the latency of a small put-with-signal round trip, through the device-initiated
layer. The numbers calibrate the algorithm cut-overs of the collective engine (which sizes are
latency bound, what one direction of NVLink carries with SM-issued traffic).

The counterpart of the reference's fabric sample (rocprofiler-compute/sample/fabric.hip:200-238:
grid-stride read / write / atomic kernels on local, host or remote-GPU memory).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m rocm_systems_b200.bench.p2p_probe --bytes 268435456 --iters 10

Device-timed with CUDA events after warm-up; every rank probes at the same time towards the peer
``(rank + d) % n`` for each distance ``d`` (the traffic pattern of a ring step, all links busy).
"""
from __future__ import annotations

import argparse
import json

import torch

from ..comm import init_from_env
from ..shmem import CMP_GE, SIGNAL_ADD, Shmem


def _timed(fn, sh, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    sh.barrier_all()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--bytes", type=int, default=256 << 20)
    ap.add_argument("--small", type=int, default=8, help="payload of the latency probe in bytes")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    comm = init_from_env()
    sh = Shmem(comm, heap_bytes=a.bytes + (16 << 20))
    n, me = sh.n_pes, sh.my_pe
    sym = sh.malloc_tensor((a.bytes,), torch.uint8)
    sig = sh.malloc_tensor((32,), torch.int64)
    sig.zero_()
    local = torch.empty(a.bytes, dtype=torch.uint8, device=comm.device)
    small = torch.zeros(max(a.small, 8), dtype=torch.uint8, device=comm.device)
    sh.barrier_all()
    rows = []
    rounds = 0
    for d in range(1, n):
        to, frm = (me + d) % n, (me - d) % n
        rounds = 0  # the signal word of this distance starts at zero
        t_put = _timed(lambda: sh.put(sym, local, to), sh, a.warmup, a.iters)
        t_get = _timed(lambda: sh.get(local, sym, to), sh, a.warmup, a.iters)
        t_dma = _timed(lambda: sh.put_dma(sym, local, to), sh, a.warmup, a.iters)   # the same bytes by copy engine, no SM
        # latency: put a few bytes with a signal to `to`, wait for the one `frm` sends here
        def ping():
            nonlocal rounds
            rounds += 1
            sh.put_signal(sym[:small.numel()], small, sig[d:d + 1], 1, to, op=SIGNAL_ADD)
            sh.wait_until(sig[d:d + 1], CMP_GE, rounds)
        t_lat = _timed(ping, sh, a.warmup, max(a.iters, 20))
        rows.append({"distance": d, "to": to, "from": frm, "put_gbs": a.bytes / t_put / 1e9, "get_gbs": a.bytes / t_get / 1e9,
                     "put_dma_gbs": a.bytes / t_dma / 1e9, "put_signal_wait_us": t_lat * 1e6})
    status = sh.take_status()
    parts = comm.host_all_gather(json.dumps({"rank": me, "status": status, "rows": rows}).encode().ljust(8192))
    if me == 0:
        allr = [json.loads(p.decode().strip()) for p in parts]
        print(f"# p2p probe, {n} PEs, {a.bytes} bytes per transfer, every PE active; GB/s per direction (min over PEs), latency max over PEs")
        print("# distance   put GB/s   get GB/s   put (copy engine) GB/s   put+signal+wait us")
        for i in range(n - 1):
            put = min(r["rows"][i]["put_gbs"] for r in allr)
            get = min(r["rows"][i]["get_gbs"] for r in allr)
            dma = min(r["rows"][i]["put_dma_gbs"] for r in allr)
            lat = max(r["rows"][i]["put_signal_wait_us"] for r in allr)
            print(f"  {i + 1:8d} {put:10.1f} {get:10.1f} {dma:18.1f} {lat:18.2f}")
        if any(r["status"] for r in allr):
            print("# a bounded wait ran out on ranks:", [r["rank"] for r in allr if r["status"]])
        if a.out:
            with open(a.out, "w") as f:
                json.dump(allr, f)
    sh.barrier_all()
    torch.cuda.synchronize()
    sh.free(sig.data_ptr())
    sh.free(sym.data_ptr())
    sh.finalize()
    comm.destroy()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
