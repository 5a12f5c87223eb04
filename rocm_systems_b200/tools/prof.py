"""Tracing launcher: run any command (one process or a multi-rank launch) with tracing on, then
collect what every process wrote into CSV / JSON / Perfetto / SQLite outputs and a statistics table.

It plays the part of the reference's ``rocprofv3`` (rocprofiler-sdk/source/bin/rocprofv3.py:
option groups, environment hand-off to the tool library, output formats, ``--stats``/``--summary``).

    python -m rocm_systems_b200.tools.prof --kernel-trace --coll-trace --stats -d out -- \\
        python -m torch.distributed.run --nproc-per-node 8 train.py

What is traced, and by which part of the package:

  --kernel-trace / --memory-copy-trace / --runtime-trace / --driver-trace / --sync-trace
        ``libb200prof.so`` (CUPTI activity records), loaded into every CUDA process of the command
        through ``CUDA_INJECTION64_PATH``;
  --coll-trace    the communication library's own tracer (host and device times per collective);
  --marker-trace  ``b200tx`` ranges the program pushes (rocm_systems_b200.utils.markers);
  --sys-sample N  a background sampler in the launcher (``tools/sysmon.py``): GPU clocks / power / temperature /
                  utilisation / memory, host CPU and memory, the command's resident set, every N ms;
  --sys-trace     all of the above;
  --host-sampling call stacks of the host threads, ``libb200sample.so`` preloaded into every process of the command
                  (CPU-time or wall-clock timer; ``--stats`` then lists functions by self and inclusive share, and
                  ``<output>.folded`` feeds a flame-graph tool).
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import subprocess
import sys
from pathlib import Path
from typing import List, Optional, Sequence

from . import tracedb

PKG = Path(__file__).resolve().parents[1]


def build_env(a: argparse.Namespace, prefix: str) -> dict:
    """The environment that turns the chosen tracing on in the children (exposed for tests)."""
    env = dict(os.environ)
    cupti = a.kernel_trace or a.memory_copy_trace or a.runtime_trace or a.driver_trace or a.sync_trace
    if cupti:
        lib = PKG / "lib" / "libb200prof.so"
        if not lib.exists():
            raise SystemExit(f"{lib} is missing: run `python -m rocm_systems_b200.utils.build`")
        env["CUDA_INJECTION64_PATH"] = str(lib)
        env["B200PROF_OUTPUT"] = prefix
        env["B200PROF_KERNEL_TRACE"] = "1" if a.kernel_trace else "0"
        env["B200PROF_MEMORY_COPY_TRACE"] = "1" if a.memory_copy_trace else "0"
        env["B200PROF_RUNTIME_TRACE"] = "1" if a.runtime_trace else "0"
        env["B200PROF_DRIVER_TRACE"] = "1" if a.driver_trace else "0"
        env["B200PROF_SYNC_TRACE"] = "1" if a.sync_trace else "0"
        if a.kernel_include_regex:
            env["B200PROF_KERNEL_FILTER"] = a.kernel_include_regex
        if a.max_records:
            env["B200PROF_MAX_RECORDS"] = str(a.max_records)
    if a.coll_trace or a.marker_trace:
        env["B200COLL_TRACE"] = "1"
        env["B200COLL_TRACE_FILE"] = prefix
        if not a.disable_signal_handlers:
            env["B200COLL_TRACE_SIGNALS"] = "1"    # a run ended by SIGTERM / SIGINT / SIGABRT still writes its marker ranges
    if a.host_sampling:
        lib = PKG / "lib" / "libb200sample.so"
        if not lib.exists():
            raise SystemExit(f"{lib} is missing: run `python -m rocm_systems_b200.utils.build`")
        old = env.get("LD_PRELOAD", "")
        env["LD_PRELOAD"] = f"{lib}:{old}" if old else str(lib)
        env["B200SAMPLE_PREFIX"] = prefix
        env["B200SAMPLE_FREQ"] = str(a.sampling_freq)
        env["B200SAMPLE_CLOCK"] = a.sampling_clock
        if not a.disable_signal_handlers:
            env["B200SAMPLE_SIGNALS"] = "1"
        if a.sampling_delay > 0:
            env["B200SAMPLE_DELAY"] = str(a.sampling_delay)
        if a.sampling_duration > 0:
            env["B200SAMPLE_DURATION"] = str(a.sampling_duration)
    if a.kokkos_trace:
        lib = PKG / "lib" / "libb200kokkosp.so"
        if not lib.exists():
            raise SystemExit(f"{lib} is missing: run `python -m rocm_systems_b200.utils.build`")
        old = env.get("KOKKOS_TOOLS_LIBS", "")
        env["KOKKOS_TOOLS_LIBS"] = f"{lib};{old}" if old else str(lib)
    if a.openmp_trace:
        lib = PKG / "lib" / "libb200ompt.so"
        if not lib.exists():
            raise SystemExit(f"{lib} is missing: run `python -m rocm_systems_b200.utils.build`")
        old = env.get("OMP_TOOL_LIBRARIES", "")
        env["OMP_TOOL_LIBRARIES"] = f"{lib}:{old}" if old else str(lib)
        env["OMP_TOOL"] = "enabled"
    if a.preload:
        old = env.get("LD_PRELOAD", "")
        env["LD_PRELOAD"] = ":".join([*a.preload, old] if old else a.preload)
    if a.tool_library:
        old = env.get("B200COLL_TOOL_LIBRARIES", "")
        env["B200COLL_TOOL_LIBRARIES"] = ":".join([*a.tool_library, old] if old else a.tool_library)
    return env


def collect(prefix: str) -> List[str]:
    """Every trace file the children left behind."""
    files = sorted(set(glob.glob(prefix + ".*_kernel_trace.csv") + glob.glob(prefix + ".*_memory_copy_trace.csv") +
                       glob.glob(prefix + ".*_cuda_api_trace.csv") + glob.glob(prefix + ".rank*.csv") + glob.glob(prefix + ".markers.*.csv") + glob.glob(prefix + ".pytrace.*.csv") + glob.glob(prefix + ".sysmon.csv") +
                       glob.glob(prefix + ".*.samples.csv")))
    return files


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="prof", description=__doc__.split("\n\n")[0], formatter_class=argparse.RawDescriptionHelpFormatter)
    g = ap.add_argument_group("tracing")
    g.add_argument("--kernel-trace", action="store_true")
    g.add_argument("--memory-copy-trace", action="store_true")
    g.add_argument("--runtime-trace", action="store_true", help="CUDA runtime API calls")
    g.add_argument("--driver-trace", action="store_true", help="CUDA driver API calls")
    g.add_argument("--sync-trace", action="store_true", help="stream/event/context synchronisation")
    g.add_argument("--coll-trace", action="store_true", help="collectives of the communication library")
    g.add_argument("--marker-trace", action="store_true", help="b200tx ranges")
    g.add_argument("--kokkos-trace", action="store_true", help="Kokkos kernels, fences, deep copies, regions and sections as marker ranges "
                   "(sets KOKKOS_TOOLS_LIBS to the connector; implies --marker-trace)")
    g.add_argument("--sys-trace", action="store_true", help="everything")
    g.add_argument("--sys-sample", type=int, default=0, metavar="PERIOD_MS",
                   help="sample GPU readings (NVML), host CPU / memory and the command's resident set in the background")
    g.add_argument("--sys-sample-fields", nargs="+", default=None, metavar="FIELD",
                   help="GPU readings to sample (names of tools/smi.py; default sm_clock power temp gpu_util mem_used); the activity fields "
                        "tensor_active, sm_active, dram_active, nvlink_tx_mibs, nvlink_rx_mibs, ... put tensor-pipe and NVLink load next to the kernels")
    g.add_argument("--host-sampling", action="store_true", help="sample the call stacks of the host threads")
    g.add_argument("--sampling-freq", type=float, default=100.0, metavar="HZ")
    g.add_argument("--sampling-clock", choices=["cpu", "wall"], default="cpu",
                   help="cpu: samples in proportion to CPU time used; wall: every thread every period, blocked ones included")
    g.add_argument("--sampling-delay", type=float, default=0.0, metavar="SECONDS")
    g.add_argument("--sampling-duration", type=float, default=0.0, metavar="SECONDS", help="sample for this long after the delay, then let the command run on unsampled (0: to the end)")
    g.add_argument("--python-trace", action="store_true", help="Python calls of the command's script as ranges (the command must be `python script.py ...`: it is "
                   "run under tools/pytrace.py); implies --marker-trace so that everything lands in one database")
    g.add_argument("--python-restrict", nargs="+", default=[], metavar="REGEX", help="with --python-trace: only functions of modules whose file matches")
    g.add_argument("--openmp-trace", action="store_true", help="OpenMP parallel regions, tasks, worksharing, barriers and target regions as marker ranges "
                   "(sets OMP_TOOL_LIBRARIES to the OMPT tool; implies --marker-trace)")
    g = ap.add_argument_group("filtering")
    g.add_argument("--kernel-include-regex", default="")
    g.add_argument("--kernel-exclude-regex", default="", help="drop kernels whose name matches (applied when the trace is imported)")
    g.add_argument("--kernel-rename", action="store_true", help="name every kernel after the innermost marker range open on its launching thread at launch "
                   "(needs --marker-trace; with --runtime-trace the launching thread and time are exact)")
    g.add_argument("--truncate-kernels", action="store_true", help="kernel names without return type, namespaces, template and call arguments")
    g.add_argument("--kernel-iteration-range", nargs="+", default=[], metavar="RANGE",
                   help="keep only these launches of every kernel, counted from 1 per kernel name: \"[3-5]\" \"8\" \"[20-]\" (applied when the trace is imported)")
    g.add_argument("--collection-period", default="", metavar="DELAY:DURATION",
                   help="keep only what started in this window after the first record (applied when the trace is imported)")
    g.add_argument("--collection-period-unit", choices=["hour", "min", "sec", "msec", "usec", "nsec"], default="msec")
    g.add_argument("--max-records", type=int, default=0, help="per kind and process")
    g = ap.add_argument_group("output")
    g.add_argument("-d", "--output-directory", default="prof_out")
    g.add_argument("-o", "--output-file", default="trace")
    g.add_argument("--output-format", nargs="+", choices=["csv", "json", "pftrace", "db"], default=["csv", "db"])
    g.add_argument("--stats", action="store_true", help="print per-kernel / per-collective statistics")
    g.add_argument("--summary", action="store_true", help="write the statistics as <output>_summary.json as well")
    g.add_argument("--summary-per-domain", action="store_true", help="statistics of every domain (kernels, copies, each API, markers, collectives) on its own")
    g.add_argument("--summary-groups", nargs="+", default=[], metavar="REGEX",
                   help="statistics over unions of domains: one regular expression on domain names per group, e.g. 'KERNEL_DISPATCH|MEMORY_COPY'")
    g.add_argument("--summary-units", choices=["sec", "msec", "usec", "nsec"], default="nsec")
    g.add_argument("--summary-output-file", default="", metavar="NAME", help="print the statistics into <output-directory>/NAME.txt instead of the terminal")
    g.add_argument("--output-config", action="store_true", help="write the options this pass ran with to <output>_config.json")
    g.add_argument("--top", type=int, default=15)
    g = ap.add_argument_group("counter collection")
    g.add_argument("--pmc", nargs="+", default=[], metavar="COUNTER",
                   help="collect these derived counters (tools/counter_defs.yaml; 'all' for every one) for the kernels of the command: the command runs "
                        "under Nsight Compute for exactly the raw metrics they need, clocks untouched; writes <output>_counter_collection.csv")
    g.add_argument("--pmc-kernel", default="", metavar="REGEX", help="kernels to capture (default: all, bounded by --pmc-count)")
    g.add_argument("--pmc-count", type=int, default=5, help="launches to capture (a capture replays every launch several times: keep it small)")
    g.add_argument("--pmc-skip", type=int, default=0, help="matching launches to skip first")
    g.add_argument("--pmc-dry-run", action="store_true", help="print the Nsight Compute command line and stop")
    g.add_argument("-L", "--list-avail", "--list-pmc", dest="list_pmc", action="store_true", help="list the derived counters and stop")
    g = ap.add_argument_group("job files")
    g.add_argument("-i", "--input", default="", metavar="FILE",
                   help="YAML or JSON file with a list `jobs:` (or a .txt file with one `pmc: COUNTER ...` line per pass and optional `kernel: NAME ...`); each job is a set of this launcher's options (long names, dashes or underscores), "
                        "run as a pass of its own into <output-directory>/pass_<n>/ with the options of the command line as defaults")
    g = ap.add_argument_group("tools")
    g.add_argument("--tool-library", action="append", default=[], help="extra dispatch-table tool(s) to load into the communication library")
    g.add_argument("--preload", action="append", default=[], metavar="LIBRARY", help="libraries to put in front of LD_PRELOAD (a sanitizer runtime, an allocator)")
    g.add_argument("--disable-signal-handlers", action="store_true",
                   help="do not flush the marker ranges when the command is ended by SIGTERM / SIGINT / SIGQUIT / SIGABRT (by default they are "
                        "written, then the signal takes its course; handlers of the program itself are never replaced)")
    g.add_argument("--echo", action="store_true", help="print the command and the environment variables this launcher sets before running")
    ap.add_argument("command", nargs=argparse.REMAINDER, help="-- command to run")
    return ap


def python_traced(cmd: Sequence[str], restrict: Sequence[str] = ()) -> Optional[List[str]]:
    """``python [interpreter options] script.py args`` (or a ``python -m torch.distributed.run ... script.py args`` launch) -> the
    same under the Python function tracer; None when the command is not of that form (``-m`` and ``-c`` have no script file)."""
    if not cmd or not os.path.basename(cmd[0]).startswith("python"):
        return None
    extra = ["-MR", *restrict] if restrict else []
    # A multi-rank launch: `python -m torch.distributed.run <its options> script.py args` runs the tracer as the module of
    # every rank (`... -m rocm_systems_b200.tools.pytrace -- script.py args`).
    if len(cmd) > 3 and cmd[1] == "-m" and cmd[2] in ("torch.distributed.run", "torch.distributed.launch"):
        for j in range(3, len(cmd)):
            if cmd[j] in ("-m", "--module", "--no-python", "--no_python"):
                return None
            if cmd[j].endswith(".py"):
                return [*cmd[:j], "-m", "rocm_systems_b200.tools.pytrace", *extra, "--", *cmd[j:]]
        return None
    i = 1
    while i < len(cmd) and cmd[i].startswith("-"):
        if cmd[i] in ("-m", "-c"):
            return None
        i += 2 if cmd[i] in ("-W", "-X") else 1
    if i >= len(cmd) or not cmd[i].endswith(".py"):
        return None
    return [*cmd[:i], "-m", "rocm_systems_b200.tools.pytrace", *extra, "--", *cmd[i:]]


def collect_counters(a, cmd: Sequence[str], prefix: str) -> int:
    """The ``--pmc`` mode: one bounded Nsight Compute run of the command for the chosen derived counters, then one row per
    (launch, counter) in ``<output>_counter_collection.csv`` (the layout of the reference launcher's counter-collection file:
    dispatch id, kernel name, counter name, value)."""
    from . import counters, roofline

    cs = counters.CounterSet.load()
    if a.pmc != ["all"]:
        known = {d["name"] for d in cs.defs}
        missing = [c for c in a.pmc if c not in known]
        if missing:
            print(f"prof: unknown counter(s): {', '.join(missing)} (see --list-pmc)", file=sys.stderr)
            return 2
        cs = counters.CounterSet([{k: v for k, v in d.items() if k != "ast"} for d in cs.defs if d["name"] in a.pmc])
    if not 1 <= a.pmc_count <= 20:
        print("prof: --pmc-count must be between 1 and 20", file=sys.stderr)
        return 2
    ncu_cmd = counters.collect_command(cs.required_metrics(), cmd, a.pmc_kernel, a.pmc_count, a.pmc_skip, prefix + "_counters")
    if a.pmc_dry_run:
        print(" ".join(ncu_cmd))
        return 0
    rc = subprocess.call(ncu_cmd)
    if rc != 0:
        print(f"prof: ncu exited with {rc}", file=sys.stderr)
        return rc
    n = write_counter_collection(cs, roofline.read_ncu(prefix + "_counters.ncu-rep"), roofline.load_peaks("MEASURED_PEAKS.json"),
                                 prefix + "_counter_collection.csv")
    print(f"prof: {n} counter values in {prefix}_counter_collection.csv", file=sys.stderr)
    return 0


def write_counter_collection(cs, kernels, peaks: dict, path: str) -> int:
    """One row per (captured launch, derived counter that could be evaluated); returns the number of rows."""
    import csv as _csv

    units = {d["name"]: d.get("unit", "") for d in cs.defs}
    n = 0
    with open(path, "w", newline="") as f:
        w = _csv.writer(f)
        w.writerow(["Dispatch_Id", "Kernel_Name", "Counter_Name", "Counter_Value", "Unit"])
        for i, k in enumerate(kernels):
            for name, v in cs.evaluate(dict(k.raw), peaks, {}).items():
                if v is not None and v == v:
                    w.writerow([i, k.name, name, f"{v:.6g}", units[name]])
                    n += 1
    return n


def load_jobs(path: str) -> List[dict]:
    """The jobs of an input file (the reference launcher's --input: several differently configured passes over one command)."""
    text = Path(path).read_text()
    if path.endswith(".json"):
        doc = json.loads(text)
    elif path.endswith(".txt"):
        # The reference's plain-text form: every `pmc:` line is one counter-collection pass; `kernel:` narrows all of them.
        passes, kernels = [], []
        for raw in text.splitlines():
            line = raw.split("#", 1)[0].strip()
            key, _, rest = line.partition(":")
            if key.strip() == "pmc" and rest.split():
                passes.append(rest.split())
            elif key.strip() == "kernel" and rest.split():
                kernels += rest.split()
        doc = {"jobs": [dict({"pmc": p}, **({"pmc_kernel": "|".join(kernels)} if kernels else {})) for p in passes]}
    else:
        import yaml

        doc = yaml.safe_load(text)
    jobs = doc.get("jobs") if isinstance(doc, dict) else doc
    if not isinstance(jobs, list) or not all(isinstance(j, dict) for j in jobs) or not jobs:
        raise ValueError(f"{path}: expected a non-empty list `jobs:` of option mappings")
    return jobs


def job_argv(job: dict) -> List[str]:
    """One job as command-line words: `kernel_trace: true` -> --kernel-trace, `pmc: [a, b]` -> --pmc a b, `top: 5` -> --top 5."""
    out: List[str] = []
    for key, val in job.items():
        flag = "--" + str(key).replace("_", "-")
        if isinstance(val, bool):
            if val:
                out.append(flag)
        elif isinstance(val, (list, tuple)):
            out += [flag, *[str(v) for v in val]]
        elif val is not None:
            out += [flag, str(val)]
    return out


def main(argv: Optional[Sequence[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    a = parser().parse_args(argv)
    if a.input:
        try:
            jobs = load_jobs(a.input)
        except (OSError, ValueError) as e:
            print(f"prof: {e}", file=sys.stderr)
            return 2
        split = argv.index("--") if "--" in argv else len(argv)
        head, tail = argv[:split], argv[split:]
        drop, keep = {"-i", "--input"}, []
        skip = False
        for w in head:          # the command line without the job file itself
            if skip:
                skip = False
                continue
            if w in drop:
                skip = True
                continue
            if w.startswith("--input="):
                continue
            keep.append(w)
        worst = 0
        for n, job in enumerate(jobs):
            words = job_argv({k: v for k, v in job.items() if k not in ("output_directory", "output-directory")})
            outdir = str(Path(job.get("output_directory", job.get("output-directory", a.output_directory))) / f"pass_{n}")
            print(f"prof: pass {n}: {' '.join(words) or '(defaults)'} -> {outdir}", file=sys.stderr)
            rc = main([*keep, *words, "-d", outdir, *tail])
            worst = worst or rc
        return worst
    cmd = a.command[1:] if a.command and a.command[0] == "--" else a.command
    if a.list_pmc:
        from . import counters

        for d in counters.CounterSet.load().defs:
            print(f"{d['name']:<30} [{d.get('panel', '')}] {d.get('unit', '')}: {d.get('description', '')}")
        return 0
    if not cmd:
        print("prof: no command given (put it after --)", file=sys.stderr)
        return 2
    if a.kokkos_trace or a.openmp_trace or a.python_trace:
        a.marker_trace = True
    if a.python_trace:
        cmd = python_traced(cmd, a.python_restrict)
        if cmd is None:
            print("prof: --python-trace needs a command of the form `python script.py [arguments]`", file=sys.stderr)
            return 2
    if a.sys_trace:
        a.kernel_trace = a.memory_copy_trace = a.runtime_trace = a.sync_trace = a.coll_trace = a.marker_trace = True
    if not (a.kernel_trace or a.memory_copy_trace or a.runtime_trace or a.driver_trace or a.sync_trace or a.coll_trace or a.marker_trace
            or a.host_sampling):
        a.kernel_trace = True
    outdir = Path(a.output_directory)
    outdir.mkdir(parents=True, exist_ok=True)
    prefix = str(outdir / a.output_file)
    if a.pmc:
        return collect_counters(a, cmd, prefix)   # a run of its own: a profiled run is not a traced or a timed one
    env = build_env(a, prefix)
    if a.echo:
        changed = {k: v for k, v in sorted(env.items()) if os.environ.get(k) != v}
        print("prof: " + " ".join(f"{k}={v}" for k, v in changed.items()) + " " + " ".join(cmd), file=sys.stderr)
    if a.output_config:
        Path(prefix + "_config.json").write_text(json.dumps({k: v for k, v in vars(a).items() if k != "command"} | {"command": list(cmd)}, indent=1))
    if a.sys_sample > 0:
        from .smi import FIELDS
        from .sysmon import GPU_FIELDS, SystemSampler

        unknown = [f for f in (a.sys_sample_fields or []) if f not in FIELDS]
        if unknown:
            print(f"prof: unknown --sys-sample-fields {unknown}; known: {', '.join(FIELDS)}", file=sys.stderr)
            return 2
        child = subprocess.Popen(cmd, env=env)
        with SystemSampler(period_ms=a.sys_sample, pids=[child.pid], gpu_fields=a.sys_sample_fields or GPU_FIELDS) as sampler:
            rc = child.wait()
        sampler.write_csv(prefix + ".sysmon.csv")
    else:
        rc = subprocess.call(cmd, env=env)
    if rc < 0:
        rc = 128 - rc     # ended by a signal: the shell's convention for the exit status
    files = collect(prefix)
    if not files:
        print("prof: the command left no trace files (did it use the GPU / the communication library?)", file=sys.stderr)
        return rc
    db_path = prefix + ".db"
    if os.path.exists(db_path):
        os.remove(db_path)
    with tracedb.TraceDB(db_path) as db:
        total = sum(db.import_csv(f, command=" ".join(cmd)) for f in files)
        if a.collection_period:
            delay, _, duration = a.collection_period.partition(":")
            to_ms = {"hour": 3.6e6, "min": 6e4, "sec": 1e3, "msec": 1.0, "usec": 1e-3, "nsec": 1e-6}[a.collection_period_unit]
            db.keep_window(float(delay or 0) * to_ms, float(duration or 0) * to_ms)
        if a.kernel_iteration_range:
            db.keep_kernel_iterations(tracedb.TraceDB.parse_iteration_ranges(a.kernel_iteration_range))
        if a.kernel_exclude_regex:
            db.drop_kernels(a.kernel_exclude_regex)
        if a.truncate_kernels:
            db.truncate_kernel_names()
        if a.kernel_rename:
            db.rename_kernels_by_marker()
        summary = db.summary(a.top)
        if a.summary_per_domain or a.summary_groups:
            extra = db.domain_summaries(a.top, a.summary_groups)
            if not a.summary_per_domain:
                extra["domains"] = {}
            summary.update(extra)
        summary = tracedb.scale_units(summary, a.summary_units)
        if "pftrace" in a.output_format:
            db.to_perfetto(prefix + ".perfetto.json")
        if "json" in a.output_format:
            out = {}
            for view in ("kernels", "regions", "collectives"):
                names, rows = db.query(f"select * from {view}")
                out[view] = [dict(zip(names, r)) for r in rows]
            Path(prefix + ".json").write_text(json.dumps(out))
        if "csv" in a.output_format:
            db.to_csv(prefix)
        if a.host_sampling:
            db.to_folded(prefix + ".folded")
    if "db" not in a.output_format:
        os.remove(db_path)
    if "csv" not in a.output_format:
        for f in files:
            os.remove(f)
    for f in glob.glob(prefix + ".*.folded"):   # per-process stacks: merged into <output>.folded above
        os.remove(f)
    if a.summary_output_file:
        with open(outdir / (a.summary_output_file + ".txt"), "w") as f:
            tracedb.print_summary(summary, file=f)
    elif a.stats or a.summary_per_domain or a.summary_groups:
        tracedb.print_summary(summary)
    if a.summary:
        Path(prefix + "_summary.json").write_text(json.dumps(summary, indent=1))
    print(f"prof: {total} records from {len(files)} file(s) under {outdir}", file=sys.stderr)
    return rc


if __name__ == "__main__":
    sys.exit(main())
