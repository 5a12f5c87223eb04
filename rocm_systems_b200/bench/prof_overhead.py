"""Tracing overhead harness: run a command several times plain and several times under the
tracing launcher with each chosen set of options, and report the slowdown.

The counterpart of the reference's ``rocprofv3-benchmark.py`` (rocprofiler-sdk/benchmark: runs a
workload under tracing configurations and stores the timings in SQLite).

    python -m rocm_systems_b200.bench.prof_overhead --repeat 3 --config kernel="--kernel-trace" \\
        --config all="--sys-trace" --db overhead.db -- python bench.py --model tiny --steps 20 --no-e2e
"""
from __future__ import annotations

import argparse
import shlex
import sqlite3
import statistics
import subprocess
import sys
import tempfile
import time
from typing import Dict, List, Optional, Sequence


def time_command(cmd: Sequence[str], repeat: int) -> List[float]:
    out = []
    for _ in range(repeat):
        t0 = time.perf_counter()
        rc = subprocess.call(cmd, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
        if rc != 0:
            raise RuntimeError(f"{' '.join(cmd)} exited with {rc}")
        out.append(time.perf_counter() - t0)
    return out


def measure(cmd: Sequence[str], configs: Dict[str, str], repeat: int) -> dict:
    base = time_command(cmd, repeat)
    res = {"command": " ".join(cmd), "repeat": repeat, "baseline_s": base, "baseline_median_s": statistics.median(base), "configs": {}}
    for name, opts in configs.items():
        with tempfile.TemporaryDirectory() as d:
            traced = [sys.executable, "-m", "rocm_systems_b200.tools.prof", *shlex.split(opts), "--output-format", "db", "-d", d, "--", *cmd]
            ts = time_command(traced, repeat)
        med = statistics.median(ts)
        res["configs"][name] = {"options": opts, "times_s": ts, "median_s": med,
                                "overhead_percent": 100.0 * (med - res["baseline_median_s"]) / res["baseline_median_s"]}
    return res


def store(db_path: str, res: dict) -> None:
    db = sqlite3.connect(db_path)
    db.execute("create table if not exists overhead(ts real, command text, config text, options text, repeat integer, median_s real,"
               " baseline_median_s real, overhead_percent real)")
    now = time.time()
    for name, c in res["configs"].items():
        db.execute("insert into overhead values (?,?,?,?,?,?,?,?)",
                   (now, res["command"], name, c["options"], res["repeat"], c["median_s"], res["baseline_median_s"], c["overhead_percent"]))
    db.commit()
    db.close()


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="prof_overhead", description=__doc__.split("\n\n")[0])
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--config", action="append", default=[], metavar="NAME=OPTIONS", help="launcher options to measure, e.g. kernel=--kernel-trace")
    ap.add_argument("--db", default="")
    ap.add_argument("command", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = a.command[1:] if a.command and a.command[0] == "--" else a.command
    if not cmd:
        ap.error("give the command after --")
    configs = dict(c.split("=", 1) for c in a.config) or {"kernel": "--kernel-trace", "all": "--sys-trace"}
    res = measure(cmd, configs, a.repeat)
    print(f"baseline {res['baseline_median_s']:.3f} s (median of {a.repeat})")
    for name, c in res["configs"].items():
        print(f"{name:<12} {c['median_s']:.3f} s  {c['overhead_percent']:+.1f} %   [{c['options']}]")
    if a.db:
        store(a.db, res)
    return 0


if __name__ == "__main__":
    sys.exit(main())
