"""List every setting of the communication library: environment names, current value, default and
meaning — what ``rocprof-sys-avail`` is to the reference's settings
(rocprofiler-systems/source/bin/rocprof-sys-avail) and ``Flag::Refresh`` is to its runtime's
(rocr-runtime/runtime/hsa-runtime/core/util/flag.h:78-299).

    python -m rocm_systems_b200.tools.avail [--json] [--changed] [--component NAME ...] [--all]

Without ``--all`` only the communication library's settings are listed (they are read from the library itself). ``--all``
adds the settings of the tool libraries and tools, which read plain environment variables: the activity tracer, the host
sampler, the causal profiler, the Kokkos connector, device management, the benchmark binaries and the model code.
``--component`` narrows to some of them (the reference's ``rocprof-sys-avail --categories``).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import sys
from typing import List, Optional, Sequence

from .. import _lib


def settings() -> List[dict]:
    lib = _lib.load()
    lib.b200collDescribeSettings.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    lib.b200collDescribeSettings.restype = ctypes.c_size_t
    need = lib.b200collDescribeSettings(None, 0)
    buf = ctypes.create_string_buffer(need)
    lib.b200collDescribeSettings(buf, need)
    return json.loads(buf.value.decode())


# (component, environment name, default, meaning). A test checks every name against the sources that read it.
TOOL_SETTINGS = [
    ("prof", "B200PROF_OUTPUT", "", "prefix of the activity tracer's files; setting it starts tracing when libb200prof.so is injected"),
    ("prof", "B200PROF_KERNEL_TRACE", "1", "kernel activity records"),
    ("prof", "B200PROF_MEMORY_COPY_TRACE", "0", "memory copy and memset records"),
    ("prof", "B200PROF_RUNTIME_TRACE", "0", "CUDA runtime API records"),
    ("prof", "B200PROF_DRIVER_TRACE", "0", "CUDA driver API records"),
    ("prof", "B200PROF_SYNC_TRACE", "0", "synchronisation records"),
    ("prof", "B200PROF_KERNEL_FILTER", "", "regular expression: keep only kernels whose name matches"),
    ("prof", "B200PROF_MAX_RECORDS", "0", "stop recording after this many records (0: no limit)"),
    ("sample", "B200SAMPLE_PREFIX", "", "prefix of the host sampler's files; setting it starts sampling when libb200sample.so is preloaded"),
    ("sample", "B200SAMPLE_FREQ", "100", "samples per second"),
    ("sample", "B200SAMPLE_CLOCK", "cpu", "cpu: threads that burn CPU time; wall: every thread every period"),
    ("sample", "B200SAMPLE_DELAY", "0", "seconds before the first sample"),
    ("sample", "B200SAMPLE_DURATION", "0", "seconds of sampling after the delay (0: until the program ends)"),
    ("sample", "B200SAMPLE_SIGNALS", "0", "1: write the samples when SIGTERM / SIGINT / SIGQUIT / SIGABRT ends the program (the launcher sets it)"),
    ("sample", "B200SAMPLE_MAX_SAMPLES", "262144", "samples kept; later ones are counted as dropped"),
    ("causal", "B200CAUSAL_FILE", "", "output of the causal profiler; setting it starts experiments when libb200causal.so is preloaded"),
    ("causal", "B200CAUSAL_BINARY_SCOPE", "%MAIN%", "regular expressions (';' between them) on the loaded objects whose functions may be selected"),
    ("causal", "B200CAUSAL_FUNCTION_SCOPE", "", "regular expressions on the functions that may be selected (empty: all in the binary scope)"),
    ("causal", "B200CAUSAL_FUNCTION_EXCLUDE", "", "regular expressions on functions never selected (names starting with _ never are)"),
    ("causal", "B200CAUSAL_SOURCE_RANGES", "", "file of address ranges per source line (written by tools/causal.py -S): select lines instead of functions"),
    ("causal", "B200CAUSAL_FIXED_SPEEDUP", "0,10,...,100", "virtual speed-ups (percent) to draw from"),
    ("causal", "B200CAUSAL_BACKEND", "auto", "sample source: perf (per-thread CPU-clock events), timer (ITIMER_PROF, one sample per scheduler tick), auto (perf if allowed)"),
    ("causal", "B200CAUSAL_FREQ", "1000", "samples per second of a thread's CPU time (timer backend: the scheduler tick is the floor)"),
    ("causal", "B200CAUSAL_EXPERIMENT_SECONDS", "0.5", "first length of an experiment; doubled while progress points are visited fewer than 10 times"),
    ("causal", "B200CAUSAL_DELAY", "0", "seconds before the first experiment"),
    ("causal", "B200CAUSAL_DURATION", "0", "seconds of experimenting (0: until the program ends)"),
    ("causal", "B200CAUSAL_END_TO_END", "0", "one experiment over the whole run"),
    ("causal", "B200CAUSAL_FILE_RESET", "0", "truncate the output instead of appending"),
    ("causal", "B200CAUSAL_RANDOM_SEED", "0", "seed of the draws (0: from the clock)"),
    ("causal", "B200CAUSAL_VERBOSE", "0", "announce every experiment on stderr"),
    ("kokkosp", "B200KOKKOSP_MEMORY_EVENTS", "0", "a marker per Kokkos allocation and deallocation"),
    ("kokkosp", "B200KOKKOSP_VERBOSE", "0", "say on stderr that the connector was loaded"),
    ("instrument", "B200INSTR_PREFIX", "", "prefix of the function statistics and coverage files; setting it switches libb200instr.so on"),
    ("instrument", "B200INSTR_MIN_US", "100", "calls at least this long become marker ranges (negative: none)"),
    ("instrument", "B200INSTR_MAX_DEPTH", "64", "calls nested deeper than this are counted, not timed"),
    ("ompt", "B200OMPT_VERBOSE", "0", "say on stderr what the OpenMP runtime offered and how many callbacks it accepted"),
    ("smi", "B200SMI_NVML_LIBRARY", "libnvidia-ml.so.1", "NVML library to load (tests point it at a stand-in)"),
    ("smi", "B200SMI_ALLOW_SET", "0", "must be 1, together with --allow-set, before any setter acts"),
    ("perf", "NCCL_TESTS_DEVICE", "", "first CUDA device of the benchmark binaries"),
    ("perf", "NCCL_TESTS_MIN_BW", "", "fail a benchmark run whose average bus bandwidth is below this (GB/s)"),
    ("perf", "NCCL_TESTS_SPLIT", "", "split the ranks into communicators: AND / OR / MOD / DIV with a number"),
    ("perf", "NCCL_TESTS_SPLIT_MASK", "", "older spelling of NCCL_TESTS_SPLIT=AND <mask>"),
    ("model", "B200COLL_CPU_AFFINITY", "0", "1: pin each rank's process to the CPUs its GPU is attached to when the process group or communicator is made"),
    ("model", "B200_LINEAR_GEMM", "", "which GEMM the model's linear layers use (own kernel by default; cublas for comparison)"),
    ("coll", "B200COLL_TOOL_REGISTER_ENABLED", "1", "0: load no tool library and hand the dispatch table to nobody"),
    ("coll", "B200COLL_TOOL_SECURE", "0", "1: only tool libraries named by an absolute path, owned by root or this user and writable by nobody else"),
    ("coll", "B200COLL_TRACE_SIGNALS", "0", "1: write the marker ranges when SIGTERM / SIGINT / SIGQUIT / SIGABRT ends the program (the launcher sets it)"),
    ("coll", "B200COLL_EMULATE_RANKS", "", "run the multi-rank kernels of the self-tests as one cooperative kernel over this many ranks"),
    ("coll", "B200COLL_SAMPLE_TOOL_OUTPUT", "", "where the example tool library writes its call log"),
]


def tool_settings() -> List[dict]:
    import os

    return [{"name": env, "env": [env], "value": os.environ.get(env, default), "default": default, "doc": doc, "component": comp}
            for comp, env, default, doc in TOOL_SETTINGS]


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="avail", description=__doc__.split("\n\n")[0])
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--changed", action="store_true", help="only settings whose value differs from the default")
    ap.add_argument("--all", action="store_true", help="also the settings of the tool libraries and tools")
    ap.add_argument("--component", nargs="+", default=None, help="only these components (coll, prof, sample, causal, kokkosp, ompt, instrument, smi, perf, model); implies --all")
    a = ap.parse_args(argv)
    rows = [dict(r, component=r.get("component", "coll")) for r in settings()]
    if a.all or a.component:
        rows += tool_settings()
    if a.component:
        rows = [r for r in rows if r["component"] in a.component]
    if a.changed:
        rows = [r for r in rows if _norm(r["value"]) != _norm(r["default"])]
    if a.json:
        print(json.dumps(rows, indent=1))
        return 0
    w = max((len(r["env"][0]) for r in rows), default=10)
    for r in rows:
        alias = f" (also {r['env'][1]})" if len(r["env"]) > 1 else ""
        print(f"{r['env'][0]:<{w}}  = {r['value'] or '\"\"':<12} default {r['default'] or '\"\"':<10} {r['doc']}{alias}")
    return 0


def _norm(v: str) -> str:
    """'64M' and '67108864' are the same value."""
    v = v.strip()
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    if v and v[-1].upper() in mult and v[:-1].replace(".", "", 1).isdigit():
        return str(int(float(v[:-1]) * mult[v[-1].upper()]))
    return v


if __name__ == "__main__":
    sys.exit(main())
