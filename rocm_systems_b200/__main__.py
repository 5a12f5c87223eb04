"""``python -m rocm_systems_b200 [tool] [arguments]``: one door to the command-line tools of the package. Without a tool
name it lists them with what each is for."""
from __future__ import annotations

import importlib
import sys

TOOLS = {
    "smi": "device management: readings, topology, processes, events, activity",
    "telemetry": "telemetry daemon and client: watches, job statistics, policies, health, Prometheus",
    "info": "devices, links and build of this machine",
    "prof": "tracing launcher: kernels, copies, APIs, collectives, markers, host samples, counters",
    "tracedb": "trace database: import, summary, query, diff, export",
    "pytrace": "Python function tracer",
    "instrument": "function statistics and coverage for code built with -finstrument-functions",
    "causal": "causal profiler of host code (virtual speed-ups)",
    "sysmon": "background sampler of GPU, host and process counters",
    "counters": "derived hardware counters, analysis report, comparison of captures",
    "roofline": "kernels on the roofline of the measured peaks",
    "avail": "settings of the library and the tools, with their current values",
    "plan": "what the collective planner would choose for a size",
    "tune": "tuning table from measured sweeps",
    "validate": "checks of a trace against expectations",
}


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        print("usage: python -m rocm_systems_b200 <tool> [arguments]\n")
        for name, what in TOOLS.items():
            print(f"  {name:<11} {what}")
        return 0
    if argv[0] == "--version":
        from . import __version__

        print(__version__)
        return 0
    if argv[0] not in TOOLS:
        print(f"unknown tool {argv[0]!r}; one of: {', '.join(TOOLS)}", file=sys.stderr)
        return 2
    mod = importlib.import_module(f"{__package__}.tools.{argv[0]}")
    return int(mod.main(argv[1:]) or 0)


if __name__ == "__main__":
    sys.exit(main())
