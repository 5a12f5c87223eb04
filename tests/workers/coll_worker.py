"""One rank of the multi-GPU collective correctness sweep (launched by torchrun or by
tests/test_gpu_collectives.py as child processes, one per GPU).

Inputs are small integers stored in the element type, so every reduction is exact in any order
and results are compared bitwise against a reduction computed locally from all ranks' seeds —
the idea of the rccl-tests verifiable oracle (rccl-tests/verifiable/verifiable.h:16-34).
"""
import argparse
import json
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402

from rocm_systems_b200 import _lib  # noqa: E402
from rocm_systems_b200.comm import init_from_env  # noqa: E402

FAILS = []
SKEW = {"ms": 0.0, "rng": None}  # --skew-ms: a random host-side pause per rank between operations


def gen(rank, n, dtype, seed, lo=-4, hi=5, device="cuda"):
    g = torch.Generator(device="cpu").manual_seed(1000 * seed + rank)
    x = torch.randint(lo, hi, (n,), generator=g, dtype=torch.int32)
    return x.to(torch.float32).to(dtype).to(device) if dtype.is_floating_point else x.to(dtype).to(device)


def reduce_ref(parts, op):
    acc = parts[0].to(torch.float64) if parts[0].dtype.is_floating_point else parts[0].to(torch.int64)
    for p in parts[1:]:
        q = p.to(acc.dtype)
        if op == "sum" or op == "avg":
            acc = acc + q
        elif op == "prod":
            acc = acc * q
        elif op == "max":
            acc = torch.maximum(acc, q)
        elif op == "min":
            acc = torch.minimum(acc, q)
    if op == "avg":
        acc = acc / len(parts) if parts[0].dtype.is_floating_point else torch.div(acc, len(parts), rounding_mode="trunc")
    return acc


def check(name, got, want):
    if SKEW["ms"] > 0:  # ranks then enter the next operation at different times (protocol races show as wrong data)
        time.sleep(SKEW["rng"].uniform(0.0, SKEW["ms"]) / 1e3)
    w = want.to(torch.float32).to(got.dtype) if got.dtype.is_floating_point else want.to(got.dtype)
    a = got.view(torch.uint8) if got.element_size() == 1 else got
    b = w.view(torch.uint8) if w.element_size() == 1 else w
    if not torch.equal(a, b):
        bad = (a != b).nonzero().flatten()
        FAILS.append(f"{name}: {bad.numel()} wrong of {got.numel()}, first at {bad[0].item()}: got {got.flatten()[bad[0]].item()} want {w.flatten()[bad[0]].item()}")
        return False
    return True


GUARD_BYTES = 256
GUARD_FILL = 0x5A


def guarded(cnt, dt, dev, lead=0):
    """A zeroed receive buffer of ``cnt`` elements with ``lead`` elements before it and 256 bytes after it filled with a
    pattern, so that a kernel writing outside its output shows up. Returns (raw bytes, output view)."""
    es = torch.empty((), dtype=dt).element_size()
    raw = torch.full(((lead + cnt) * es + GUARD_BYTES,), GUARD_FILL, dtype=torch.uint8, device=dev)
    raw[lead * es:(lead + cnt) * es] = 0
    return raw, raw[:(lead + cnt) * es].view(dt)[lead:]


def check_guards(name, raw, cnt, dt, lead=0):
    es = torch.empty((), dtype=dt).element_size()
    front, back = raw[:lead * es], raw[(lead + cnt) * es:]
    if not (bool((front == GUARD_FILL).all()) and bool((back == GUARD_FILL).all())):
        FAILS.append(f"{name}/guard: {int((front != GUARD_FILL).sum()) + int((back != GUARD_FILL).sum())} bytes outside the output were written")


def set_algo(lib, algo):
    if algo == "auto":
        os.environ.pop("B200COLL_ALGO", None)
    else:
        os.environ["B200COLL_ALGO"] = algo
    lib.b200collRefreshFlags()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--skew-ms", type=float, default=0.0, help="random pause per rank between operations, up to this many ms")
    args = ap.parse_args()
    comm = init_from_env()
    if args.skew_ms > 0:
        import random

        SKEW["ms"], SKEW["rng"] = args.skew_ms, random.Random(977 * comm.rank + 1)
    lib = _lib.load()
    rank, n = comm.rank, comm.nranks
    dev = comm.device
    results = {"nranks": n, "nvls": comm.nvls, "cases": 0}
    algos = ["auto", "p2p"] + (["nvls"] if comm.nvls else [])
    dtypes = [torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64, torch.uint8, torch.float64]
    if hasattr(torch, "float8_e4m3fn"):
        dtypes += [torch.float8_e4m3fn, torch.float8_e5m2]
    sizes = [1, 3, 257, 4099, 70001, 1 << 20] if args.quick else [1, 3, 257, 4099, 70001, (1 << 20) + 5, 20 * (1 << 20) + 8]
    seed = 0
    t0 = time.time()
    for algo in algos:
        set_algo(lib, algo)
        for dt in dtypes:
            es = torch.empty((), dtype=dt).element_size()
            ops = ["sum", "max", "min", "avg", "prod"]
            for cnt in sizes:
                if es == 8 and cnt > (1 << 20) + 5:
                    continue
                for op in ops:
                    if op != "sum" and cnt > 70001:
                        continue
                    seed += 1
                    lo, hi = (-4, 5)
                    if op == "prod":
                        lo, hi = (1, 3)
                    if dt == torch.uint8:
                        lo = max(lo, 0)
                    parts = [gen(r, cnt, dt, seed, lo, hi) for r in range(n)]
                    want = reduce_ref(parts, op)
                    # all_reduce out of place (misaligned by one element) and in place
                    raw, out = guarded(cnt, dt, dev, lead=1)
                    comm.all_reduce(parts[rank], out, op=op)
                    check(f"all_reduce/{algo}/{dt}/{op}/{cnt}/oop", out, want)
                    check_guards(f"all_reduce/{algo}/{dt}/{op}/{cnt}/oop", raw, cnt, dt, lead=1)
                    inp = parts[rank].clone()
                    comm.all_reduce(inp, op=op)
                    check(f"all_reduce/{algo}/{dt}/{op}/{cnt}/inplace", inp, want)
                    results["cases"] += 2
                    if op in ("sum", "max") and cnt >= n:
                        # reduce_scatter: every rank contributes n*per elements
                        per = cnt // n
                        if per:
                            full = [p[: per * n] for p in parts]
                            w = reduce_ref(full, op)[rank * per:(rank + 1) * per]
                            raw, o = guarded(per, dt, dev)
                            comm.reduce_scatter(full[rank].clone(), o, op=op)
                            check(f"reduce_scatter/{algo}/{dt}/{op}/{per}", o, w)
                            check_guards(f"reduce_scatter/{algo}/{dt}/{op}/{per}", raw, per, dt)
                            # in place: recv is the rank's slice of send
                            s2 = full[rank].clone()
                            comm.reduce_scatter(s2, s2[rank * per:(rank + 1) * per], op=op)
                            check(f"reduce_scatter/{algo}/{dt}/{op}/{per}/inplace", s2[rank * per:(rank + 1) * per], w)
                            results["cases"] += 2
                        for root in sorted({0, n - 1}):
                            o = torch.zeros(cnt, dtype=torch.float32, device=dev).to(dt) if dt.is_floating_point else torch.zeros(cnt, dtype=dt, device=dev)
                            comm.reduce(parts[rank], o if rank == root else None, root=root, op=op)
                            if rank == root:
                                check(f"reduce/{algo}/{dt}/{op}/{cnt}/root{root}", o, want)
                            results["cases"] += 1
                if dt in (torch.float32, torch.bfloat16, torch.uint8):
                    for cnt in sizes:
                        seed += 1
                        parts = [gen(r, cnt, dt, seed, 0, 100) for r in range(n)]
                        raw, o = guarded(cnt * n, dt, dev)
                        comm.all_gather(parts[rank], o)
                        check(f"all_gather/{algo}/{dt}/{cnt}", o, torch.cat(parts).to(torch.float64 if dt.is_floating_point else torch.int64))
                        check_guards(f"all_gather/{algo}/{dt}/{cnt}", raw, cnt * n, dt)
                        o2 = o.clone().zero_()
                        o2[rank * cnt:(rank + 1) * cnt] = parts[rank]
                        comm.all_gather(o2[rank * cnt:(rank + 1) * cnt], o2)
                        check(f"all_gather/{algo}/{dt}/{cnt}/inplace", o2, torch.cat(parts).to(torch.float64 if dt.is_floating_point else torch.int64))
                        for root in sorted({0, n - 1}):
                            b = parts[root].clone() if rank == root else torch.zeros_like(parts[0])
                            comm.broadcast(b, root=root)
                            check(f"broadcast/{algo}/{dt}/{cnt}/root{root}", b, parts[root].to(torch.float64 if dt.is_floating_point else torch.int64))
                        results["cases"] += 4
    torch.cuda.synchronize()
    results["coll_seconds"] = time.time() - t0

    # PreMulSum: rank r multiplies by (r + 1)
    set_algo(lib, "auto")
    for dt in (torch.float32, torch.bfloat16):
        for cnt in (5, 4099, (1 << 20) + 5):
            seed += 1
            parts = [gen(r, cnt, dt, seed) for r in range(n)]
            op = comm.premul_sum(float(rank + 1), dt)
            o = torch.zeros_like(parts[0])
            comm.all_reduce(parts[rank], o, op=op)
            want = sum((r + 1) * parts[r].to(torch.float64) for r in range(n))
            check(f"premulsum/{dt}/{cnt}", o, want)
            torch.cuda.synchronize()
            comm.redop_destroy(op)
            results["cases"] += 1

    # Point-to-point family
    for dt in (torch.float32, torch.bfloat16):
        for cnt in (1, 1000, 300007, 3 * (1 << 20) + 1):
            seed += 1
            parts = [gen(r, cnt * n, dt, seed, 0, 100) for r in range(n)]
            raw, o = guarded(cnt * n, dt, dev)
            comm.all_to_all(parts[rank], o)
            want = torch.cat([parts[s][rank * cnt:(rank + 1) * cnt] for s in range(n)])
            check(f"all_to_all/{dt}/{cnt}", o, want.to(torch.float64))
            check_guards(f"all_to_all/{dt}/{cnt}", raw, cnt * n, dt)
            # ring send/recv
            raw, r_buf = guarded(cnt, dt, dev)
            comm.group_start()
            comm.send(parts[rank][:cnt], (rank + 1) % n)
            comm.recv(r_buf, (rank - 1) % n)
            comm.group_end()
            check(f"sendrecv/{dt}/{cnt}", r_buf, parts[(rank - 1) % n][:cnt].to(torch.float64))
            check_guards(f"sendrecv/{dt}/{cnt}", raw, cnt, dt)
            # gather / scatter
            g = torch.zeros(cnt * n, dtype=dt, device=dev) if rank == 0 else None
            comm.gather(parts[rank][:cnt], g, root=0)
            if rank == 0:
                check(f"gather/{dt}/{cnt}", g, torch.cat([parts[s][:cnt] for s in range(n)]).to(torch.float64))
            sc = torch.zeros(cnt, dtype=dt, device=dev)
            comm.scatter(parts[n - 1] if rank == n - 1 else None, sc, root=n - 1)
            check(f"scatter/{dt}/{cnt}", sc, parts[n - 1][rank * cnt:(rank + 1) * cnt].to(torch.float64))
            results["cases"] += 4
    # all_to_allv with uneven counts: rank s sends (s + d + 1) * 100 elements to rank d
    cnts = [[(s + d + 1) * 100 for d in range(n)] for s in range(n)]
    seed += 1
    parts = [gen(r, sum(cnts[r]), torch.float32, seed, 0, 100) for r in range(n)]
    sd = [sum(cnts[rank][:d]) for d in range(n)]
    rc = [cnts[s][rank] for s in range(n)]
    rd = [sum(rc[:s]) for s in range(n)]
    o = torch.zeros(sum(rc), dtype=torch.float32, device=dev)
    comm.all_to_allv(parts[rank], cnts[rank], sd, o, rc, rd)
    want = torch.cat([parts[s][sum(cnts[s][:rank]):sum(cnts[s][:rank]) + cnts[s][rank]] for s in range(n)])
    check("all_to_allv", o, want.to(torch.float64))
    results["cases"] += 1

    # Symmetric windows: zero-copy paths
    for algo in algos:
        set_algo(lib, algo)
        for dt in (torch.float32, torch.bfloat16):
            es = torch.empty((), dtype=dt).element_size()
            cnt = 3 * (1 << 20)
            sym = comm.sym_alloc(2 * cnt * es * 2)
            seed += 1
            parts = [gen(r, cnt, dt, seed) for r in range(n)]
            s_t = sym.tensor((cnt,), dt)
            r_t = sym.tensor((cnt,), dt, offset_bytes=cnt * es)
            s_t.copy_(parts[rank])
            comm.all_reduce(s_t, r_t)
            check(f"sym_all_reduce/{algo}/{dt}", r_t, reduce_ref(parts, "sum"))
            s_t.copy_(parts[rank])
            comm.all_reduce(s_t)
            check(f"sym_all_reduce_inplace/{algo}/{dt}", s_t, reduce_ref(parts, "sum"))
            per = cnt // n
            s_t.copy_(parts[rank])
            o = torch.zeros(per, dtype=dt, device=dev)
            comm.reduce_scatter(s_t[: per * n], o)
            check(f"sym_reduce_scatter/{algo}/{dt}", o, reduce_ref([p[: per * n] for p in parts], "sum")[rank * per:(rank + 1) * per])
            s_t[:per].copy_(parts[rank][:per])
            og = torch.zeros(per * n, dtype=dt, device=dev)
            comm.all_gather(s_t[:per], og)
            check(f"sym_all_gather/{algo}/{dt}", og, torch.cat([p[:per] for p in parts]).to(torch.float64))
            if rank == 1 % n:
                r_t.copy_(parts[rank])
            else:
                r_t.zero_()
            comm.broadcast(r_t, root=1 % n)
            check(f"sym_broadcast/{algo}/{dt}", r_t, parts[1 % n].to(torch.float64))
            torch.cuda.synchronize()
            sym.free()
            results["cases"] += 5
    set_algo(lib, "auto")

    # Sub-communicators
    if n >= 2:
        sub = comm.split(rank % 2, rank)
        x = torch.full((1000,), float(rank + 1), device=dev)
        sub.all_reduce(x)
        members = [r for r in range(n) if r % 2 == rank % 2]
        check("split_all_reduce", x, torch.full((1000,), float(sum(m + 1 for m in members)), dtype=torch.float64, device=dev))
        torch.cuda.synchronize()
        sub.destroy()
        results["cases"] += 1

    # Tracer: device stamps exist and are ordered
    comm.trace_enable(True)
    x = torch.ones(1 << 20, device=dev)
    for _ in range(3):
        comm.all_reduce(x)
    recs = comm.trace_records()
    ok = len(recs) == 3 and all(r["devEndNs"] > r["devBeginNs"] > 0 for r in recs)
    if not ok:
        FAILS.append(f"tracer: {recs}")
    results["trace_us"] = [(r["devEndNs"] - r["devBeginNs"]) / 1e3 for r in recs]
    comm.trace_enable(False)

    torch.cuda.synchronize()
    err = comm.async_error()
    if err != 0:
        FAILS.append(f"async error {err}: {comm.last_error()}")
    results["fails"] = FAILS[:20]
    results["nfails"] = len(FAILS)
    # every rank reports; rank 0 writes
    flags = comm.host_all_gather(bytes([1 if FAILS else 0]))
    anyfail = any(f[0] for f in flags)
    if args.out and rank == 0:
        Path(args.out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.out).write_text(json.dumps(results, indent=1))
    if FAILS:
        print(f"[rank {rank}] {len(FAILS)} FAILURES:\n  " + "\n  ".join(FAILS[:10]), flush=True)
    elif rank == 0:
        print(f"coll_worker OK: {results['cases']} cases on {n} ranks, nvls={comm.nvls}, {results['coll_seconds']:.1f}s", flush=True)
    comm.destroy()
    sys.exit(1 if anyfail else 0)


if __name__ == "__main__":
    main()
