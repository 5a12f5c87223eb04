"""Function-level tracing and coverage of code built with ``-finstrument-functions``.

    python -m rocm_systems_b200.tools.instrument flags                     # what to add to the compile line
    python -m rocm_systems_b200.tools.instrument run -o out/app [--min-us 50] [--trace] -- ./app args
    python -m rocm_systems_b200.tools.instrument report out/app [--top 20] [--coverage] [--json]

``run`` preloads ``libb200instr.so`` (and, with ``--trace``, the marker library, so that calls lasting at least ``--min-us``
become ranges in ``<prefix>.markers.<pid>.csv`` for the trace database); ``report`` merges the ``<prefix>.<pid>.functions.csv``
and ``<prefix>.<pid>.coverage.json`` files of all processes of the run into one table of functions by inclusive time and one
coverage figure. It stands where the reference has ``rocprof-sys-instrument`` (rocprofiler-systems
source/bin/rocprof-sys-instrument: entry / exit instrumentation of a binary, with a coverage mode, by rewriting it); here
the compiler inserts the calls, so what is covered is what was rebuilt with the flag.
"""
from __future__ import annotations

import argparse
import csv
import glob
import json
import os
import subprocess
import sys
from pathlib import Path
from typing import Dict, List, Optional, Sequence

FLAGS = "-finstrument-functions -finstrument-functions-exclude-file-list=/usr/include,/usr/lib,/usr/local/cuda"


def libraries(trace: bool) -> List[str]:
    from ..utils import build

    lib = build.build_instrument()
    if lib is None:
        raise SystemExit("libb200instr.so cannot be built here")
    out = [str(lib)]
    if trace:
        out.append(str(build.build_lib()))
    return out


def environment(prefix: str, min_us: float, max_depth: int, trace: bool) -> dict:
    env = dict(os.environ)
    old = env.get("LD_PRELOAD", "")
    env["LD_PRELOAD"] = ":".join([*libraries(trace), old] if old else libraries(trace))
    env["B200INSTR_PREFIX"] = str(Path(prefix).resolve())
    env["B200INSTR_MIN_US"] = str(min_us if trace else -1)
    env["B200INSTR_MAX_DEPTH"] = str(max_depth)
    if trace:
        env["B200COLL_TRACE"] = "1"
        env.setdefault("B200COLL_TRACE_FILE", str(Path(prefix).resolve()))
    return env


def merge(prefix: str) -> dict:
    """``{"functions": [{function, calls, inclusive_ns, exclusive_ns}], "coverage": {functions_defined, functions_called,
    percent, uncalled}, "processes": n}`` over every process that wrote files with this prefix. A function counts as called
    when any process called it."""
    acc: Dict[str, List[int]] = {}
    files = sorted(glob.glob(glob.escape(prefix) + ".*.functions.csv"))
    for f in files:
        with open(f, newline="") as fh:
            for r in csv.DictReader(fh):
                a = acc.setdefault(r["function"], [0, 0, 0])
                a[0] += int(r["calls"])
                a[1] += int(r["inclusive_ns"])
                a[2] += int(r["exclusive_ns"])
    functions = [{"function": k, "calls": v[0], "inclusive_ns": v[1], "exclusive_ns": v[2]} for k, v in sorted(acc.items(), key=lambda kv: -kv[1][1])]
    defined, uncalled = 0, None
    for f in sorted(glob.glob(glob.escape(prefix) + ".*.coverage.json")):
        doc = json.loads(Path(f).read_text())
        defined = max(defined, doc["functions_defined"])
        uncalled = set(doc["uncalled"]) if uncalled is None else uncalled & set(doc["uncalled"])
    uncalled = sorted(uncalled or [])
    called = max(0, defined - len(uncalled))
    return {"functions": functions, "processes": len(files),
            "coverage": {"functions_defined": defined, "functions_called": called, "percent": round(100.0 * called / defined, 2) if defined else 0.0,
                         "uncalled": uncalled}}


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="instrument", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("flags", help="print the compiler flags that insert the entry / exit calls")
    r = sub.add_parser("run", help="run a program built with those flags")
    r.add_argument("-o", "--output", default="instr/run", metavar="PREFIX")
    r.add_argument("--min-us", type=float, default=100.0, help="with --trace: calls at least this long become marker ranges")
    r.add_argument("--max-depth", type=int, default=64, help="calls nested deeper are counted, not timed")
    r.add_argument("--trace", action="store_true", help="record long calls as marker ranges too")
    r.add_argument("--report", action="store_true", help="print the report when the program ends")
    r.add_argument("command", nargs=argparse.REMAINDER)
    p = sub.add_parser("report", help="functions by inclusive time and coverage, over all processes of a run")
    p.add_argument("prefix")
    p.add_argument("--top", type=int, default=20)
    p.add_argument("--coverage", action="store_true", help="list the functions that were never called")
    p.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    if a.cmd == "flags":
        print(FLAGS)
        return 0
    if a.cmd == "run":
        cmd = a.command[1:] if a.command and a.command[0] == "--" else a.command
        if not cmd:
            raise SystemExit("no command after --")
        Path(a.output).parent.mkdir(parents=True, exist_ok=True)
        rc = subprocess.call(cmd, env=environment(a.output, a.min_us, a.max_depth, a.trace))
        if a.report:
            main(["report", a.output])
        return rc
    doc = merge(a.prefix)
    if a.json:
        print(json.dumps(doc, indent=1))
        return 0
    from .tracedb import format_table

    if not doc["processes"]:
        print(f"instrument: no files with prefix {a.prefix}", file=sys.stderr)
        return 1
    rows = doc["functions"][:a.top]
    print(format_table(["function", "calls", "inclusive_ms", "exclusive_ms"], [[r["function"], r["calls"], r["inclusive_ns"] / 1e6, r["exclusive_ns"] / 1e6] for r in rows]))
    c = doc["coverage"]
    print(f"\ncoverage: {c['functions_called']} of {c['functions_defined']} functions called ({c['percent']} %), {doc['processes']} process(es)")
    if a.coverage:
        for name in c["uncalled"]:
            print("  never called: " + name)
    return 0


if __name__ == "__main__":
    sys.exit(main())
