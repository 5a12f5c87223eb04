"""Show what the collective planner chooses — algorithm, CTAs, pipeline chunks — for a range of
message sizes, without a GPU. It asks the library itself (``b200collPlanDry``), so the
environment (``B200COLL_ALGO``, ``NCCL_MAX_CTAS``, ``B200COLL_TUNING_FILE``, ...) applies as it
would to a real communicator.

    python -m rocm_systems_b200.tools.plan --nranks 8 --coll all_reduce -b 1K -e 1G -f 4
    B200COLL_TUNING_FILE=tuning.json python -m rocm_systems_b200.tools.plan --nranks 4 --coll reduce_scatter
"""
from __future__ import annotations

import argparse
import ctypes
import sys
from typing import Optional, Sequence

from .. import _lib

COLLS = {"all_reduce": 0, "reduce_scatter": 1, "reduce": 2, "all_gather": 3, "broadcast": 4, "alltoall": 5}
ALGOS = {1: "flag-in-data", 2: "peer loads/stores", 3: "in-switch", 4: "send/recv FIFOs"}
DTYPES = {"int8": (0, 1), "uint8": (1, 1), "int32": (2, 4), "uint32": (3, 4), "int64": (4, 8), "uint64": (5, 8), "half": (6, 2), "float": (7, 4),
          "double": (8, 8), "bfloat16": (9, 2)}
OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}


class Info(ctypes.Structure):
    _fields_ = [("algo", ctypes.c_int), ("ctas", ctypes.c_int), ("direct", ctypes.c_int), ("chunks", ctypes.c_ulonglong)]


def _size(s: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(float(s[:-1]) * mult[s[-1].upper()]) if s[-1].upper() in mult else int(s)


def plan(nranks: int, nvls: bool, coll: str, count: int, dtype: str = "float", op: str = "sum") -> dict:
    lib = _lib.load()
    lib.b200collPlanDry.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.POINTER(Info)]
    i = Info()
    _lib.check(lib.b200collPlanDry(nranks, 1 if nvls else 0, COLLS[coll], count, DTYPES[dtype][0], OPS[op], ctypes.byref(i)), "b200collPlanDry")
    return {"algo": ALGOS.get(i.algo, str(i.algo)), "ctas": i.ctas, "chunks": int(i.chunks), "direct": bool(i.direct)}


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="plan", description=__doc__.split("\n\n")[0])
    ap.add_argument("--nranks", type=int, default=8)
    ap.add_argument("--no-nvls", action="store_true", help="plan for a box without multicast")
    ap.add_argument("--coll", default="all_reduce", choices=sorted(COLLS))
    ap.add_argument("-d", "--dtype", default="float", choices=sorted(DTYPES))
    ap.add_argument("-o", "--op", default="sum", choices=sorted(OPS))
    ap.add_argument("-b", "--minbytes", default="1K")
    ap.add_argument("-e", "--maxbytes", default="1G")
    ap.add_argument("-f", "--stepfactor", type=int, default=4)
    a = ap.parse_args(argv)
    es = DTYPES[a.dtype][1]
    size, top = _size(a.minbytes), _size(a.maxbytes)
    print(f"# {a.coll}, {a.nranks} ranks, {a.dtype} {a.op}, multicast {'no' if a.no_nvls else 'yes'}; bytes are per-rank counts for all_gather / reduce_scatter and per pair for alltoall")
    print(f"{'bytes':>14}  {'algorithm':<14} {'CTAs':>5} {'chunks':>7}")
    while size <= top:
        p = plan(a.nranks, not a.no_nvls, a.coll, max(1, size // es), a.dtype, a.op)
        print(f"{size:>14}  {p['algo']:<14} {p['ctas']:>5} {p['chunks']:>7}")
        size *= max(2, a.stepfactor)
    return 0


if __name__ == "__main__":
    sys.exit(main())
