"""Causal profiling front end: run a program under ``libb200causal.so`` and turn its experiments into predictions
"making function F x % faster makes the program y % faster".

    python -m rocm_systems_b200.tools.causal run -o exp.coz -n 3 -- ./app args        # experiments drawn while the program runs
    python -m rocm_systems_b200.tools.causal run -o exp.coz -e -n 5 -s 0 10 20 30 -F cpu_slow_func -- ./app args
    python -m rocm_systems_b200.tools.causal report exp.coz [--json] [--point iteration] [--min-experiments 2]
    python -m rocm_systems_b200.tools.causal report exp.coz --validate cpu_slow_func iteration 20 20 5

``run`` is the counterpart of the reference's ``rocprof-sys-causal`` launcher (rocprofiler-systems
source/bin/rocprof-sys-causal/rocprof-sys-causal.cpp: ``-n`` iterations, ``-e`` end-to-end runs with one fixed experiment
each, ``-s`` speed-ups, ``-F`` / ``-B`` function and binary scopes, ``-S`` source scope, ``-d`` delay, ``-t`` duration):
with ``-e`` every (function or source scope, speed-up) pair is run ``-n`` times. With ``-S`` the line table of the
executable is decoded here (``readelf --debug-dump=decodedline``) and the address ranges of the chosen lines are handed to
the library, which then selects lines instead of functions. ``report`` restates what its ``tests/validate-causal-json.py`` computes:
per selected function and progress point, the time per visit at each virtual speed-up against the time per visit at
speed-up 0 of the same function, with the spread over the experiments, and ``--validate`` checks predictions against
expected values with a tolerance (exit code 1 on a miss), the way the reference's end-to-end tests do.

The program marks progress with ``B200CAUSAL_PROGRESS`` / ``B200CAUSAL_BEGIN`` / ``B200CAUSAL_END``
(``include/b200coll/causal.h``) or, from Python, ``rocm_systems_b200.utils.causal.progress``.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
from collections import defaultdict
from pathlib import Path
from typing import Dict, Iterable, List, Optional


def library() -> Path:
    from ..utils import build

    lib = build.build_causal()
    if lib is None:
        raise SystemExit("libb200causal.so cannot be built here")
    return lib


# ---------------------------------------------------------------------------------------------------------------- parse
def parse(text: str) -> List[dict]:
    """Experiments of one output file: ``{selected, speedup (percent), duration (ns, pauses taken out), real_duration,
    selected_samples, throughput: {name: visits}, latency: {name: {arrivals, departures, difference}}}``."""
    out: List[dict] = []
    cur: Optional[dict] = None
    for line in text.splitlines():
        parts = line.rstrip("\n").split("\t")
        kind, kv = parts[0], {}
        for p in parts[1:]:
            k, _, v = p.partition("=")
            kv[k] = v
        if kind == "experiment":
            cur = {"selected": kv.get("selected", ""), "speedup": int(round(float(kv.get("speedup", 0)) * 100)),
                   "duration": int(kv.get("duration", 0)), "real_duration": int(kv.get("real-duration", kv.get("duration", 0))),
                   "selected_samples": int(kv.get("selected-samples", 0)), "throughput": {}, "latency": {}}
            out.append(cur)
        elif kind in ("throughput-point", "progress-point") and cur is not None:
            cur["throughput"][kv.get("name", "")] = int(kv.get("delta", 0))
        elif kind == "latency-point" and cur is not None:
            cur["latency"][kv.get("name", "")] = {k: int(kv.get(k, 0)) for k in ("arrivals", "departures", "difference")}
        elif kind in ("startup", "runtime"):
            cur = None
    return out


def _mean(xs: Iterable[float]) -> float:
    xs = list(xs)
    return sum(xs) / len(xs) if xs else 0.0


def _std(xs: Iterable[float]) -> float:
    xs = list(xs)
    if len(xs) < 2:
        return 0.0
    m = _mean(xs)
    return math.sqrt(sum((x - m) ** 2 for x in xs) / len(xs))


def analyze(experiments: List[dict], point: Optional[str] = None, min_experiments: int = 1) -> List[dict]:
    """One entry per (selected function, progress point) that has a baseline (speed-up 0): ``{selected, point, kind,
    baseline_period_ns, rows: [{speedup, program_speedup, stddev, experiments}], impact}``. For a latency point the period is
    the time an item spends in flight where that can be told (Little's law), else the time per departure. The program speed-up at s is
    ``100 * (1 - period_s / period_0)`` with ``period = sum(duration) / sum(visits)`` over the experiments at s; the spread
    is that of the per-experiment speed-ups; ``impact`` is the area under the curve per unit of virtual speed-up (what the
    reference sorts by)."""
    groups: Dict[tuple, Dict[int, List[tuple]]] = defaultdict(lambda: defaultdict(list))
    for e in experiments:
        for name, visits in e["throughput"].items():
            if visits > 0:
                groups[(e["selected"], name, "throughput")][e["speedup"]].append((visits, e["duration"]))
        for name, lat in e["latency"].items():
            if lat["departures"] > 0:
                # (departures, duration, items in flight when the experiment ended, arrivals)
                groups[(e["selected"], name, "latency")][e["speedup"]].append((lat["departures"], e["duration"], max(lat["difference"], 0), lat["arrivals"]))
    out = []
    for (selected, name, kind), by in sorted(groups.items()):
        if point is not None and name != point:
            continue
        if 0 not in by:
            continue
        # A latency point with items in flight at the ends of its experiments gives the time an item spends between begin and
        # end by Little's law: items in flight (averaged over the experiments, weighted by their length) / arrival rate
        # = sum(in flight x duration) / sum(arrivals). Where nothing was in flight when the experiments ended (whole runs,
        # strictly sequential items) the time per departure is what is left to compare.
        little = kind == "latency" and all(sum(r[2] * r[1] for r in runs) > 0 and sum(r[3] for r in runs) > 0 for runs in by.values())

        def period_of(runs):
            if little:
                return sum(r[2] * r[1] for r in runs) / sum(r[3] for r in runs)
            return sum(r[1] for r in runs) / sum(r[0] for r in runs)

        def one(r):
            return (r[2] * r[1] / r[3]) if (little and r[3]) else r[1] / r[0]

        base = period_of(by[0])
        base_spread = _std([100.0 * (1.0 - one(r) / base) for r in by[0]])
        rows = []
        for s in sorted(by):
            runs = by[s]
            if len(runs) < min_experiments:
                continue
            rows.append({"speedup": s, "program_speedup": 100.0 * (1.0 - period_of(runs) / base),
                         "stddev": _std([100.0 * (1.0 - one(r) / base) for r in runs]), "experiments": len(runs)})
        area = sum(0.5 * (a["program_speedup"] + b["program_speedup"]) * (b["speedup"] - a["speedup"]) for a, b in zip(rows, rows[1:]))
        span = rows[-1]["speedup"] - rows[0]["speedup"] if len(rows) > 1 else 0
        out.append({"selected": selected, "point": name, "kind": kind + (" (time in flight)" if little else ""), "baseline_period_ns": base, "baseline_stddev": base_spread, "rows": rows,
                    "impact": area / span if span else 0.0})
    out.sort(key=lambda r: -r["impact"])
    return out


def format_report(results: List[dict]) -> str:
    lines = []
    for r in results:
        lines.append(f"{r['selected']}  [{r['kind']} point: {r['point']}]  time per visit at speed-up 0: {r['baseline_period_ns'] / 1e6:.3f} ms"
                     f"  impact {r['impact']:.1f}")
        lines.append(f"  {'virtual speed-up %':>18} {'program speed-up %':>19} {'+/-':>7} {'experiments':>12}")
        for row in r["rows"]:
            lines.append(f"  {row['speedup']:>18d} {row['program_speedup']:>19.1f} {row['stddev']:>7.1f} {row['experiments']:>12d}")
    return "\n".join(lines) if lines else "no function has experiments at speed-up 0 and at another speed-up"


def validate(results: List[dict], checks: List[tuple]) -> List[str]:
    """``checks``: (function substring, point, virtual speed-up, expected program speed-up, tolerance). The tolerance is
    widened by the spread of the baseline and of the prediction, as the reference does on shared machines. Returns the
    failures as text."""
    bad = []
    for func, point, s, expected, tol in checks:
        rows = [(r, row) for r in results if func in r["selected"] and r["point"] == point for row in r["rows"] if row["speedup"] == s]
        if not rows:
            bad.append(f"{func} / {point} / {s} %: no experiment")
            continue
        for r, row in rows:
            allowed = tol + max(r["baseline_stddev"], row["stddev"])
            if abs(row["program_speedup"] - expected) > allowed:
                bad.append(f"{r['selected']} / {point} / {s} %: predicted {row['program_speedup']:.1f} %, expected {expected:.1f} +/- {allowed:.1f}")
    return bad


# -------------------------------------------------------------------------------------------------------- source lines
def decode_line_table(text: str) -> List[tuple]:
    """Rows of ``readelf --debug-dump=decodedline -W``: ``(path, line, lo, hi)`` for every non-empty address range, where
    ``path`` is the heading the rows stand under (as the compiler recorded it) and ``hi`` is the address of the next row
    of the same sequence."""
    rows: List[tuple] = []          # (path, line or None at the end of a sequence, address)
    path = ""
    for raw in text.splitlines():
        line = raw.rstrip()
        if not line or line.startswith("Contents of") or line.startswith("File name"):
            continue
        if line.endswith(":") and "0x" not in line:
            path = line[:-1]
            if path.startswith("CU: "):
                path = path[4:]
            continue
        parts = line.split()
        if len(parts) < 3 or not parts[2].startswith("0x"):
            continue
        rows.append((path, None if parts[1] == "-" else int(parts[1]), int(parts[2], 16)))
    out = []
    for (p, ln, addr), (_, _, nxt) in zip(rows, rows[1:]):
        if ln is not None and nxt > addr:
            out.append((p, ln, addr, nxt))
    return out


def source_ranges(exe: str, patterns: List[str]) -> Dict[str, List[tuple]]:
    """Address ranges per source line (``"file.cc:123"``) of ``exe`` for the lines whose ``path:line`` matches one of the
    regular expressions (a bare file pattern selects every line of the file). Needs debug information (``-g``)."""
    import re

    r = subprocess.run(["readelf", "--debug-dump=decodedline", "-W", exe], capture_output=True, text=True)
    if r.returncode != 0:
        raise SystemExit(f"readelf failed on {exe}: {r.stderr.strip()}")
    res = [re.compile(p) for p in patterns]
    merged: Dict[str, List[tuple]] = defaultdict(list)
    for path, ln, lo, hi in decode_line_table(r.stdout):
        key = f"{path}:{ln}"
        if not any(x.search(key) for x in res):
            continue
        name = f"{os.path.basename(path)}:{ln}"
        spans = merged[name]
        if spans and spans[-1][1] == lo:
            spans[-1] = (spans[-1][0], hi)
        else:
            spans.append((lo, hi))
    return dict(merged)


def write_source_ranges(path: Path, ranges: Dict[str, List[tuple]]) -> None:
    with open(path, "w") as f:
        for name, spans in sorted(ranges.items()):
            f.write(name + "\t" + ",".join(f"{lo:x}-{hi:x}" for lo, hi in sorted(spans)) + "\n")


# ------------------------------------------------------------------------------------------------------------------ run
def environment(a, speedup: Optional[int] = None, function: Optional[str] = None, source: Optional[str] = None) -> dict:
    env = dict(os.environ)
    lib = str(library())
    env["LD_PRELOAD"] = lib + (":" + env["LD_PRELOAD"] if env.get("LD_PRELOAD") else "")
    env["B200CAUSAL_FILE"] = str(Path(a.output).resolve())
    if a.binary_scope:
        env["B200CAUSAL_BINARY_SCOPE"] = ";".join(a.binary_scope)
    scope = [function] if function is not None else a.function_scope
    if scope:
        env["B200CAUSAL_FUNCTION_SCOPE"] = ";".join(scope)
    if a.function_exclude:
        env["B200CAUSAL_FUNCTION_EXCLUDE"] = ";".join(a.function_exclude)
    sources = [source] if source is not None else a.source_scope
    if sources:
        import shutil

        exe = shutil.which(a.command[0]) or a.command[0]
        ranges = source_ranges(exe, sources)
        if not ranges:
            raise SystemExit(f"no line of {exe} matches {sources} (is it built with -g?)")
        table = Path(str(Path(a.output).resolve()) + ".ranges")
        write_source_ranges(table, ranges)
        env["B200CAUSAL_SOURCE_RANGES"] = str(table)
        env.pop("B200CAUSAL_FUNCTION_SCOPE", None)
    speedups = [speedup] if speedup is not None else a.speedups
    if speedups:
        env["B200CAUSAL_FIXED_SPEEDUP"] = ",".join(str(s) for s in speedups)
    env["B200CAUSAL_BACKEND"] = a.backend
    env["B200CAUSAL_FREQ"] = str(a.freq)
    env["B200CAUSAL_EXPERIMENT_SECONDS"] = str(a.experiment_seconds)
    env["B200CAUSAL_DELAY"] = str(a.delay)
    env["B200CAUSAL_DURATION"] = str(a.duration)
    env["B200CAUSAL_END_TO_END"] = "1" if a.end_to_end else "0"
    if a.seed:
        env["B200CAUSAL_RANDOM_SEED"] = str(a.seed)
    if a.verbose:
        env["B200CAUSAL_VERBOSE"] = "1"
    return env


def plan(a) -> List[dict]:
    """The runs ``run`` will make: ``-n`` plain runs, or with ``-e`` one per (function scope, speed-up, iteration)."""
    if not a.end_to_end:
        return [{"speedup": None, "function": None, "source": None} for _ in range(a.iterations)]
    speedups = a.speedups or [0, 10, 20, 30, 40, 50]
    if a.source_scope:
        return [{"speedup": s, "function": None, "source": src} for _ in range(a.iterations) for src in a.source_scope for s in speedups]
    functions = a.function_scope or [None]
    return [{"speedup": s, "function": f, "source": None} for _ in range(a.iterations) for f in functions for s in speedups]


def cmd_run(a) -> int:
    if not a.command:
        raise SystemExit("no command after --")
    Path(a.output).parent.mkdir(parents=True, exist_ok=True)
    if a.reset and Path(a.output).exists():
        Path(a.output).unlink()
    rc = 0
    for i, job in enumerate(plan(a)):
        env = environment(a, job["speedup"], job["function"], job["source"])
        if a.verbose:
            print(f"[causal] run {i + 1}: function scope {job['function'] or a.function_scope or 'all'}, speed-ups {job['speedup'] if job['speedup'] is not None else a.speedups or 'default'}",
                  file=sys.stderr)
        r = subprocess.run(a.command, env=env)
        rc = rc or r.returncode
    if a.report and Path(a.output).exists():
        print(format_report(analyze(parse(Path(a.output).read_text()))))
    return rc


def cmd_report(a) -> int:
    experiments: List[dict] = []
    for f in a.files:
        experiments += parse(Path(f).read_text())
    results = analyze(experiments, a.point, a.min_experiments)
    if a.json:
        print(json.dumps({"experiments": len(experiments), "results": results}, indent=1))
    else:
        print(f"{len(experiments)} experiments")
        print(format_report(results))
    if a.validate:
        if len(a.validate) % 5:
            raise SystemExit("--validate takes groups of five: FUNCTION POINT SPEEDUP EXPECTED TOLERANCE")
        v = a.validate
        checks = [(v[i], v[i + 1], int(v[i + 2]), float(v[i + 3]), float(v[i + 4])) for i in range(0, len(v), 5)]
        bad = validate(results, checks)
        for b in bad:
            print("FAILED " + b, file=sys.stderr)
        return 1 if bad else 0
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="b200-causal", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run", help="run a command under the causal profiler")
    r.add_argument("-o", "--output", default="causal/experiments.coz")
    r.add_argument("-n", "--iterations", type=int, default=1)
    r.add_argument("-e", "--end-to-end", action="store_true", help="one experiment per run, over the whole run")
    r.add_argument("-s", "--speedups", type=int, nargs="*", default=[])
    r.add_argument("-F", "--function-scope", nargs="*", default=[], help="regular expressions on function names")
    r.add_argument("-FE", "--function-exclude", nargs="*", default=[])
    r.add_argument("-S", "--source-scope", nargs="*", default=[], help="regular expressions on <path>:<line> of the executable's line table "
                   "(\"solver.cc:120\", or \"solver.cc\" for every line of it): experiments select source lines instead of functions")
    r.add_argument("-B", "--binary-scope", nargs="*", default=[], help="regular expressions on the paths of loaded objects (default: the executable)")
    r.add_argument("-d", "--delay", type=float, default=0.0, help="seconds before the first experiment")
    r.add_argument("-t", "--duration", type=float, default=0.0, help="seconds of experimenting; 0 = the whole run")
    r.add_argument("--backend", choices=["auto", "perf", "timer"], default="auto",
                   help="sample source: per-thread CPU-clock events (perf: samples at --freq), the process CPU-time timer (timer: one sample per "
                        "scheduler tick), or perf where the kernel allows it and timer otherwise (auto)")
    r.add_argument("--freq", type=float, default=1000.0)
    r.add_argument("--experiment-seconds", type=float, default=0.5)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("-r", "--reset", action="store_true", help="start from an empty output file")
    r.add_argument("--report", action="store_true", help="print the predictions after the runs")
    r.add_argument("-v", "--verbose", action="store_true")
    r.add_argument("command", nargs=argparse.REMAINDER)
    p = sub.add_parser("report", help="predictions from one or more output files")
    p.add_argument("files", nargs="+")
    p.add_argument("--point", default=None)
    p.add_argument("--min-experiments", type=int, default=1)
    p.add_argument("--json", action="store_true")
    p.add_argument("--validate", nargs="*", default=[], metavar="FUNCTION POINT SPEEDUP EXPECTED TOLERANCE")
    a = ap.parse_args(argv)
    if a.cmd == "run":
        if a.command and a.command[0] == "--":
            a.command = a.command[1:]
        return cmd_run(a)
    return cmd_report(a)


if __name__ == "__main__":
    sys.exit(main())
