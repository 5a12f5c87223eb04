"""Validators for trace outputs: check that a Perfetto JSON, a trace database or a trace CSV is well
formed and contains what a test expects (categories, slice names, counter tracks, minimum counts).

The counterpart of the reference's output validators (rocprofiler-systems/tests/validate-perfetto-proto.py
and the readers under rocprofiler-sdk/tests/pytest-packages/pytest_utils): tests run an application
under the tracer and then point a validator at the files.

    python -m rocm_systems_b200.tools.validate perfetto trace.perfetto.json --category kernel --min-slices 10 --counter gpu_power
    python -m rocm_systems_b200.tools.validate db trace.db --table kernel_dispatch:10 --table collective:1
    python -m rocm_systems_b200.tools.validate csv out.rank0.csv --column Device_Us --function ncclAllReduce
    python -m rocm_systems_b200.tools.validate causal exp.coz --min-experiments 8 --selected cpu_slow_func --point iteration
"""
from __future__ import annotations

import argparse
import csv
import json
import sqlite3
import sys
from typing import List, Optional, Sequence


def check_perfetto(path: str, categories: Sequence[str] = (), names: Sequence[str] = (), counters: Sequence[str] = (), min_slices: int = 0,
                   min_flows: int = 0) -> List[str]:
    errs: List[str] = []
    try:
        doc = json.load(open(path))
    except (OSError, ValueError) as e:
        return [f"{path}: not readable JSON ({e})"]
    ev = doc.get("traceEvents")
    if not isinstance(ev, list):
        return [f"{path}: no traceEvents array"]
    slices = [e for e in ev if e.get("ph") == "X"]
    for e in slices:
        if not all(k in e for k in ("name", "ts", "dur", "pid")):
            errs.append(f"slice without name/ts/dur/pid: {e}")
            break
        if e["dur"] < 0:
            errs.append(f"negative duration in slice {e['name']!r}")
            break
    if len(slices) < min_slices:
        errs.append(f"{len(slices)} slices, expected at least {min_slices}")
    have_cat = {e.get("cat") for e in slices}
    for c in categories:
        if c not in have_cat:
            errs.append(f"no slice of category {c!r} (have {sorted(x for x in have_cat if x)})")
    for n in names:
        if not any(n in e.get("name", "") for e in slices):
            errs.append(f"no slice whose name contains {n!r}")
    tracks = {e.get("name", "") for e in ev if e.get("ph") == "C"}
    for c in counters:
        if not any(t.startswith(c) for t in tracks):
            errs.append(f"no counter track starting with {c!r} (have {sorted(tracks)[:8]})")
    # arrows: every start has its finish, the finish is not earlier, and there are as many as expected
    starts = {e.get("id"): e for e in ev if e.get("ph") == "s"}
    ends = {e.get("id"): e for e in ev if e.get("ph") == "f"}
    if set(starts) != set(ends):
        errs.append(f"{len(set(starts) ^ set(ends))} arrows without their other end")
    if any(ends[i]["ts"] < starts[i]["ts"] for i in starts if i in ends):
        errs.append("an arrow points back in time")
    if len(starts) < min_flows:
        errs.append(f"{len(starts)} arrows, expected at least {min_flows}")
    # slices on one track must not partially overlap (nesting is fine): a sign of mixed clocks
    by_track = {}
    for e in slices:
        by_track.setdefault((e["pid"], e.get("tid")), []).append((e["ts"], e["ts"] + e["dur"]))
    for key, spans in by_track.items():
        spans.sort()
        stack: List[float] = []
        for s, t in spans:
            while stack and stack[-1] <= s:
                stack.pop()
            if stack and t > stack[-1] + 1e-3:
                errs.append(f"slices on track {key} overlap without nesting")
                break
            stack.append(t)
    return errs


def check_db(path: str, tables: Sequence[str] = ()) -> List[str]:
    errs: List[str] = []
    try:
        db = sqlite3.connect(f"file:{path}?mode=ro", uri=True)
        have = {r[0] for r in db.execute("select name from sqlite_master where type in ('table', 'view')")}
    except sqlite3.Error as e:
        return [f"{path}: {e}"]
    for spec in tables:
        name, _, n = spec.partition(":")
        if name not in have:
            errs.append(f"no table or view {name!r}")
            continue
        rows = db.execute(f"select count(*) from {name}").fetchone()[0]
        if rows < int(n or 0):
            errs.append(f"{name}: {rows} rows, expected at least {n}")
    for name in ("kernel_dispatch", "region", "collective"):
        if name in have:
            col = "device_start_ns" if name == "collective" else "start_ns"
            end = "device_end_ns" if name == "collective" else "end_ns"
            bad = db.execute(f"select count(*) from {name} where {end} < {col}").fetchone()[0]
            if bad:
                errs.append(f"{name}: {bad} rows end before they start")
    db.close()
    return errs


def check_csv(path: str, columns: Sequence[str] = (), functions: Sequence[str] = (), min_rows: int = 1) -> List[str]:
    errs: List[str] = []
    try:
        rows = list(csv.DictReader(open(path, newline="")))
    except OSError as e:
        return [f"{path}: {e}"]
    if len(rows) < min_rows:
        errs.append(f"{len(rows)} rows, expected at least {min_rows}")
    if rows:
        for c in columns:
            if c not in rows[0]:
                errs.append(f"no column {c!r} (have {list(rows[0])})")
        for fn in functions:
            key = "Function" if "Function" in rows[0] else "Kernel_Name"
            if not any(fn in r.get(key, "") for r in rows):
                errs.append(f"no row whose {key} contains {fn!r}")
        if "Start_Timestamp" in rows[0] and any(int(r["End_Timestamp"]) < int(r["Start_Timestamp"]) for r in rows):
            errs.append("a row ends before it starts")
    return errs


def check_causal(path: str, min_experiments: int = 1, selected: Sequence[str] = (), points: Sequence[str] = ()) -> List[str]:
    """An output file of the causal profiler: experiments are there, have sane durations and a speed-up between 0 and 100 %,
    the named functions were selected and the named progress points were visited."""
    import re

    from .causal import parse

    errs: List[str] = []
    try:
        ex = parse(open(path).read())
    except OSError as e:
        return [f"{path}: {e}"]
    if len(ex) < min_experiments:
        errs.append(f"{len(ex)} experiments, expected at least {min_experiments}")
    for e in ex:
        if not 0 <= e["speedup"] <= 100 or e["duration"] <= 0 or e["duration"] > e["real_duration"]:
            errs.append(f"experiment on {e['selected']!r}: speed-up {e['speedup']} %, duration {e['duration']} of {e['real_duration']} ns")
            break
    for pat in selected:
        if not any(re.search(pat, e["selected"]) for e in ex):
            errs.append(f"no experiment selected a function matching {pat!r}")
    for name in points:
        if not any(e["throughput"].get(name, 0) > 0 or e["latency"].get(name, {}).get("departures", 0) > 0 for e in ex):
            errs.append(f"progress point {name!r} was never visited during an experiment")
    return errs


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="validate", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="kind", required=True)
    p = sub.add_parser("perfetto")
    p.add_argument("file")
    p.add_argument("--category", action="append", default=[])
    p.add_argument("--name", action="append", default=[])
    p.add_argument("--counter", action="append", default=[])
    p.add_argument("--min-slices", type=int, default=0)
    p.add_argument("--min-flows", type=int, default=0, help="arrows from a host call to the device work it started")
    p = sub.add_parser("db")
    p.add_argument("file")
    p.add_argument("--table", action="append", default=[], metavar="NAME[:MIN_ROWS]")
    p = sub.add_parser("csv")
    p.add_argument("file")
    p.add_argument("--column", action="append", default=[])
    p.add_argument("--function", action="append", default=[])
    p.add_argument("--min-rows", type=int, default=1)
    p = sub.add_parser("causal")
    p.add_argument("file")
    p.add_argument("--min-experiments", type=int, default=1)
    p.add_argument("--selected", action="append", default=[], metavar="REGEX")
    p.add_argument("--point", action="append", default=[])
    a = ap.parse_args(argv)
    if a.kind == "perfetto":
        errs = check_perfetto(a.file, a.category, a.name, a.counter, a.min_slices, a.min_flows)
    elif a.kind == "causal":
        errs = check_causal(a.file, a.min_experiments, a.selected, a.point)
    elif a.kind == "db":
        errs = check_db(a.file, a.table)
    else:
        errs = check_csv(a.file, a.column, a.function, a.min_rows)
    for e in errs:
        print("FAIL:", e)
    if not errs:
        print("ok")
    return 1 if errs else 0


if __name__ == "__main__":
    sys.exit(main())
