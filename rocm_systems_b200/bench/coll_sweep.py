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


def make_ops(comm, coll: str, s: torch.Tensor, r: torch.Tensor, per: int, in_place: bool = False):
    """The call of this library and the stock NCCL call (through ``torch.distributed``) for one collective on the same
    buffers: ``s`` / ``r`` hold ``count`` elements, ``per`` is the per-rank part of the scattering / gathering ones.
    ``in_place`` uses the in-place convention of the C API (all_gather: the rank's part inside the receive buffer;
    reduce_scatter: the result inside the send buffer; all_reduce and broadcast: one buffer)."""
    rank = comm.rank
    if coll == "all_reduce":
        if in_place:
            return (lambda: comm.all_reduce(s, s)), (lambda: dist.all_reduce(s))
        return (lambda: comm.all_reduce(s, r)), (lambda: dist.all_reduce(s))
    if coll == "reduce_scatter":
        out = s[rank * per:(rank + 1) * per] if in_place else r[:per]
        return (lambda: comm.reduce_scatter(s, out)), (lambda: dist.reduce_scatter_tensor(out, s))
    if coll == "all_gather":
        src = r[rank * per:(rank + 1) * per] if in_place else s[:per]
        return (lambda: comm.all_gather(src, r)), (lambda: dist.all_gather_into_tensor(r, src))
    if coll == "broadcast":
        if in_place:
            return (lambda: comm.broadcast(s, s, root=0)), (lambda: dist.broadcast(s, 0))
        return (lambda: comm.broadcast(s, r, root=0)), (lambda: dist.broadcast(s, 0))
    if coll == "alltoall":
        return (lambda: comm.all_to_all(s, r)), (lambda: dist.all_to_all_single(r, s))
    raise SystemExit(f"unknown collective {coll}")


def sweep(comm, colls, sizes, dt: torch.dtype, send_all: torch.Tensor, recv_all: torch.Tensor, warmup: int, iters: int, nccl: bool = True,
          in_place: bool = False, on_row=None) -> list:
    """Time every (collective, size) on this library and, when ``nccl``, on stock NCCL; rccl-tests columns per row."""
    n = comm.nranks
    es = torch.empty((), dtype=dt).element_size()
    rows = []
    for coll in colls:
        for size in sizes:
            count = max(size // es, 1)
            per = count
            if coll in ("reduce_scatter", "all_gather", "alltoall"):
                per = max(count // n, 1)
                count = per * n
            s, r = send_all[:count], recv_all[:count]
            ours, ref = make_ops(comm, coll, s, r, per, in_place)
            it = iters if size <= (64 << 20) else max(iters // 4, 3)
            t_ours = time_op(ours, warmup, it)
            t_ref = time_op(ref, warmup, it) if nccl else float("nan")
            nbytes = count * es
            f = busbw_factor(coll, n)
            row = {"coll": coll, "bytes": nbytes, "count": count, "in_place": in_place, "ours_us": t_ours, "nccl_us": t_ref,
                   "ours_algbw": nbytes / t_ours / 1e3, "ours_busbw": nbytes / t_ours / 1e3 * f,
                   "nccl_algbw": nbytes / t_ref / 1e3, "nccl_busbw": nbytes / t_ref / 1e3 * f}
            rows.append(row)
            if on_row:
                on_row(row)
    return rows


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("-b", "--minbytes", default="8")
    ap.add_argument("-e", "--maxbytes", default="256M")
    ap.add_argument("-f", "--stepfactor", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--dtype", default="float", help="float, bfloat16 or half; several separated by commas")
    ap.add_argument("--colls", default="all_reduce,reduce_scatter,all_gather,broadcast,alltoall")
    ap.add_argument("--symmetric", type=int, default=0, help="1: buffers in symmetric (registered) memory")
    ap.add_argument("--placement", default="out", help="out, in or both: out-of-place and / or in-place buffers")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    comm = init_from_env()
    rank, n = comm.rank, comm.nranks
    dist.init_process_group("nccl" if not args.no_nccl else "gloo", device_id=comm.device if not args.no_nccl else None)
    lo, hi = parse_size(args.minbytes), parse_size(args.maxbytes)
    sizes = []
    size = lo
    while size <= hi:
        sizes.append(size)
        size *= args.stepfactor
    if args.symmetric:
        sym = comm.sym_alloc(2 * hi + 4096)
        send_raw = sym.tensor((hi,), torch.uint8)
        recv_raw = sym.tensor((hi,), torch.uint8, offset_bytes=hi)
    else:
        send_raw = torch.empty(hi, dtype=torch.uint8, device="cuda")
        recv_raw = torch.empty(hi, dtype=torch.uint8, device="cuda")
    rows = []
    placements = {"out": [False], "in": [True], "both": [False, True]}[args.placement]
    for dname in args.dtype.split(","):
        dt = {"float": torch.float32, "bfloat16": torch.bfloat16, "half": torch.float16}[dname]
        send_all, recv_all = send_raw.view(dt), recv_raw.view(dt)
        send_all.normal_()
        for in_place in placements:
            if rank == 0:
                print(f"# nranks {n} dtype {dname} nvls {comm.nvls} symmetric {args.symmetric} in_place {int(in_place)} warmup {args.warmup} iters {args.iters}")
                print(f"# {'coll':<15}{'size(B)':>12}{'count':>12}{'ours us':>11}{'algbw':>9}{'busbw':>9}{'nccl us':>11}{'algbw':>9}{'busbw':>9}{'ratio':>7}")

            def show(row):
                if rank == 0:
                    print(f"  {row['coll']:<15}{row['bytes']:>12}{row['count']:>12}{row['ours_us']:>11.2f}{row['ours_algbw']:>9.2f}{row['ours_busbw']:>9.2f}"
                          f"{row['nccl_us']:>11.2f}{row['nccl_algbw']:>9.2f}{row['nccl_busbw']:>9.2f}{row['nccl_us'] / row['ours_us']:>7.2f}", flush=True)

            for row in sweep(comm, args.colls.split(","), sizes, dt, send_all, recv_all, args.warmup, args.iters, not args.no_nccl, in_place, show):
                row["dtype"] = dname
                rows.append(row)
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
