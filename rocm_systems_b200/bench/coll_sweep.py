"""Collective bandwidth sweep, one process per GPU (run under torchrun):

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        -m rocm_systems_b200.bench.coll_sweep -b 8 -e 1G -f 4 --out sweep.json

For every collective and size it times this library and, side by side, stock NCCL through
``torch.distributed`` on the same buffers, and prints the rccl-tests columns (size, count, type,
time, algbw, busbw; rccl-tests/src/common.cpp:1846-1875) for both. Times are device times
(CUDA events around ``iters`` back-to-back calls), the maximum over ranks. busbw factors follow
rccl-tests: all_reduce 2(n-1)/n; all_gather, reduce_scatter, alltoall (n-1)/n; broadcast, reduce 1
(rccl-tests/src/all_reduce.cpp:48-52, all_gather.cpp:57, reduce_scatter.cpp:55, alltoall.cpp:59,
broadcast.cpp:51).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch
import torch.distributed as dist

from ..comm import init_from_env


def parse_size(s: str) -> int:
    s = s.strip()
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}.get(s[-1].upper())
    return int(float(s[:-1]) * mult) if mult else int(s)


def busbw_factor(coll: str, n: int) -> float:
    if coll == "all_reduce":
        return 2.0 * (n - 1) / n
    if coll in ("all_gather", "reduce_scatter", "alltoall"):
        return (n - 1) / n
    return 1.0


def time_op(fn, warmup: int, iters: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) * 1e3 / iters
    t = torch.tensor([us], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("-b", "--minbytes", default="8")
    ap.add_argument("-e", "--maxbytes", default="256M")
    ap.add_argument("-f", "--stepfactor", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--dtype", default="float")
    ap.add_argument("--colls", default="all_reduce,reduce_scatter,all_gather,broadcast,alltoall")
    ap.add_argument("--symmetric", type=int, default=0, help="1: buffers in symmetric (registered) memory")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    comm = init_from_env()
    rank, n = comm.rank, comm.nranks
    dist.init_process_group("nccl" if not args.no_nccl else "gloo", device_id=comm.device if not args.no_nccl else None)
    dt = {"float": torch.float32, "bfloat16": torch.bfloat16, "half": torch.float16}[args.dtype]
    es = torch.empty((), dtype=dt).element_size()
    lo, hi = parse_size(args.minbytes), parse_size(args.maxbytes)
    maxel = hi // es
    if args.symmetric:
        sym = comm.sym_alloc(2 * hi + 4096)
        send_all = sym.tensor((maxel,), dt)
        recv_all = sym.tensor((maxel,), dt, offset_bytes=hi)
    else:
        send_all = torch.empty(maxel, dtype=dt, device="cuda")
        recv_all = torch.empty(maxel, dtype=dt, device="cuda")
    send_all.normal_()
    rows = []
    if rank == 0:
        print(f"# nranks {n} dtype {args.dtype} nvls {comm.nvls} symmetric {args.symmetric} warmup {args.warmup} iters {args.iters}")
        print(f"# {'coll':<15}{'size(B)':>12}{'count':>12}{'ours us':>11}{'algbw':>9}{'busbw':>9}{'nccl us':>11}{'algbw':>9}{'busbw':>9}{'ratio':>7}")
    size = lo
    sizes = []
    while size <= hi:
        sizes.append(size)
        size *= args.stepfactor
    for coll in args.colls.split(","):
        for size in sizes:
            count = max(size // es, 1)
            if coll in ("reduce_scatter", "all_gather", "alltoall"):
                per = max(count // n, 1)
                count = per * n
            s, r = send_all[:count], recv_all[:count]
            if coll == "all_reduce":
                ours = lambda: comm.all_reduce(s, r)
                ref = lambda: dist.all_reduce(s)
            elif coll == "reduce_scatter":
                ours = lambda: comm.reduce_scatter(s, r[:per])
                ref = lambda: dist.reduce_scatter_tensor(r[:per], s)
            elif coll == "all_gather":
                ours = lambda: comm.all_gather(s[:per], r)
                ref = lambda: dist.all_gather_into_tensor(r, s[:per])
            elif coll == "broadcast":
                ours = lambda: comm.broadcast(s, s, root=0)
                ref = lambda: dist.broadcast(s, 0)
            elif coll == "alltoall":
                ours = lambda: comm.all_to_all(s, r)
                ref = lambda: dist.all_to_all_single(r, s)
            else:
                raise SystemExit(f"unknown collective {coll}")
            iters = args.iters if size <= (64 << 20) else max(args.iters // 4, 3)
            t_ours = time_op(ours, args.warmup, iters)
            t_ref = time_op(ref, args.warmup, iters) if not args.no_nccl else float("nan")
            nbytes = count * es
            f = busbw_factor(coll, n)
            row = {"coll": coll, "bytes": nbytes, "count": count, "ours_us": t_ours, "nccl_us": t_ref,
                   "ours_algbw": nbytes / t_ours / 1e3, "ours_busbw": nbytes / t_ours / 1e3 * f,
                   "nccl_algbw": nbytes / t_ref / 1e3, "nccl_busbw": nbytes / t_ref / 1e3 * f}
            rows.append(row)
            if rank == 0:
                print(f"  {coll:<15}{nbytes:>12}{count:>12}{t_ours:>11.2f}{row['ours_algbw']:>9.2f}{row['ours_busbw']:>9.2f}"
                      f"{t_ref:>11.2f}{row['nccl_algbw']:>9.2f}{row['nccl_busbw']:>9.2f}{t_ref / t_ours:>7.2f}", flush=True)
    err = comm.async_error()
    if rank == 0 and args.out:
        Path(args.out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.out).write_text(json.dumps({"nranks": n, "dtype": args.dtype, "nvls": comm.nvls, "symmetric": args.symmetric,
                                               "async_error": err, "rows": rows}, indent=1))
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    comm.destroy()
    sys.exit(1 if err else 0)


if __name__ == "__main__":
    main()
