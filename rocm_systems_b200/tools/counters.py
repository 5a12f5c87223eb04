"""Derived counters: named expressions over raw profiler metrics, defined in YAML and evaluated per
kernel launch.

The counterpart of the reference's counter service (rocprofiler-sdk/source/lib/rocprofiler-sdk/counters:
YAML definitions, an expression parser — ``parser/scanner.l`` and ``parser.y`` — and AST
evaluation in ``evaluate_ast.cpp``). The raw values here come from Nsight Compute's raw page
(``ncu -i FILE --page raw --csv``) instead of hardware counter blocks; the grammar is

    expr   := term (('+' | '-') term)*
    term   := unary (('*' | '/') unary)*
    unary  := '-' unary | atom
    atom   := NUMBER | IDENT | IDENT '(' expr (',' expr)* ')' | '(' expr ')'
    IDENT  := letters, digits, '_' and '.', e.g. dram__bytes_read.sum, peak.hbm_gbs, arg.flops

with the functions ``min``, ``max``, ``abs``, ``sqrt`` and ``select(cond, a, b)`` (a when cond is non-zero).

    python -m rocm_systems_b200.tools.counters raw.csv --peaks MEASURED_PEAKS.json --arg flops=1.0995e12

Collection (the counterpart of the reference's counter collection service, which programs the hardware blocks for the
counters a definition needs): ``--collect`` runs a command under Nsight Compute asking for exactly the raw metrics the
chosen definitions read, one kernel pattern and a bounded number of launches, and evaluates the result:

    python -m rocm_systems_b200.tools.counters --collect -k gemmPairKernel -c 2 --counter tensor_active_pct --counter hbm_gbs \
        -- python -m rocm_systems_b200.bench.kernel_cases --case gemm

``--analyze`` turns a report into the per-kernel analysis the reference's rocprofiler-compute prints (its "analyze" mode:
panels of derived metrics per dispatch): the counters grouped by panel, the warp stall reasons ranked, and a one-line
verdict on what bounds the launch:

    python -m rocm_systems_b200.tools.counters prof.ncu-rep --analyze --peaks MEASURED_PEAKS.json
    python -m rocm_systems_b200.tools.counters before.ncu-rep --compare after.ncu-rep --min-change 5 --kernel-filter gemm

The capture never locks the GPU's clocks (``--clock-control none``) and is bounded by ``-k`` / ``-c``; ``--print-command``
shows the ``ncu`` line without running anything.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import re
import sys
from pathlib import Path
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union

Node = Union[Tuple[str, float], Tuple[str, str], Tuple[str, str, list], Tuple[str, "Node"], Tuple[str, str, "Node", "Node"]]
_TOKEN = re.compile(r"\s*(?:(\d+\.?\d*(?:[eE][+-]?\d+)?|\.\d+(?:[eE][+-]?\d+)?)|([A-Za-z_][A-Za-z0-9_.]*)|(.))")
FUNCS: Dict[str, Callable[..., float]] = {
    "min": lambda *a: min(a), "max": lambda *a: max(a), "abs": lambda x: abs(x), "sqrt": lambda x: math.sqrt(x),
    "select": lambda c, a, b: a if c != 0 else b,
}


class ParseError(ValueError):
    pass


def tokenize(text: str) -> List[Tuple[str, str]]:
    out, pos = [], 0
    while pos < len(text):
        m = _TOKEN.match(text, pos)
        if not m or m.end() == pos:
            break
        pos = m.end()
        num, ident, op = m.groups()
        if num is not None:
            out.append(("num", num))
        elif ident is not None:
            out.append(("id", ident))
        elif op.strip():
            if op not in "+-*/(),":
                raise ParseError(f"unexpected character {op!r} in {text!r}")
            out.append(("op", op))
    return out


class Parser:
    def __init__(self, text: str):
        self.text, self.toks, self.i = text, tokenize(text), 0

    def peek(self) -> Tuple[str, str]:
        return self.toks[self.i] if self.i < len(self.toks) else ("end", "")

    def take(self, kind: Optional[str] = None, value: Optional[str] = None) -> Tuple[str, str]:
        t = self.peek()
        if (kind and t[0] != kind) or (value and t[1] != value):
            raise ParseError(f"expected {value or kind} at token {self.i} of {self.text!r}, found {t[1]!r}")
        self.i += 1
        return t

    def parse(self):
        node = self.expr()
        if self.peek()[0] != "end":
            raise ParseError(f"trailing input {self.peek()[1]!r} in {self.text!r}")
        return node

    def expr(self):
        node = self.term()
        while self.peek() in (("op", "+"), ("op", "-")):
            op = self.take()[1]
            node = ("bin", op, node, self.term())
        return node

    def term(self):
        node = self.unary()
        while self.peek() in (("op", "*"), ("op", "/")):
            op = self.take()[1]
            node = ("bin", op, node, self.unary())
        return node

    def unary(self):
        if self.peek() == ("op", "-"):
            self.take()
            return ("neg", self.unary())
        return self.atom()

    def atom(self):
        kind, val = self.peek()
        if kind == "num":
            self.take()
            return ("num", float(val))
        if kind == "id":
            self.take()
            if self.peek() == ("op", "("):
                self.take()
                args = [self.expr()]
                while self.peek() == ("op", ","):
                    self.take()
                    args.append(self.expr())
                self.take("op", ")")
                if val not in FUNCS:
                    raise ParseError(f"unknown function {val!r} in {self.text!r}")
                return ("call", val, args)
            return ("id", val)
        if (kind, val) == ("op", "("):
            self.take()
            node = self.expr()
            self.take("op", ")")
            return node
        raise ParseError(f"unexpected {val or 'end of input'!r} in {self.text!r}")


def parse(text: str):
    return Parser(text).parse()


def identifiers(node) -> List[str]:
    k = node[0]
    if k == "id":
        return [node[1]]
    if k == "bin":
        return identifiers(node[2]) + identifiers(node[3])
    if k == "neg":
        return identifiers(node[1])
    if k == "call":
        return [i for a in node[2] for i in identifiers(a)]
    return []


def evaluate(node, env: Dict[str, float]) -> float:
    """Evaluates an AST; a missing identifier raises KeyError, a division by zero gives NaN."""
    k = node[0]
    if k == "num":
        return node[1]
    if k == "id":
        return float(env[node[1]])
    if k == "neg":
        return -evaluate(node[1], env)
    if k == "bin":
        a, b = evaluate(node[2], env), evaluate(node[3], env)
        if node[1] == "+":
            return a + b
        if node[1] == "-":
            return a - b
        if node[1] == "*":
            return a * b
        return a / b if b != 0 else float("nan")
    if k == "call":
        return float(FUNCS[node[1]](*[evaluate(a, env) for a in node[2]]))
    raise ValueError(k)


class CounterSet:
    """Named derived metrics, each an expression over raw Nsight Compute metrics, peaks and user arguments."""

    def __init__(self, defs: Sequence[dict]):
        self.defs = []
        seen = set()
        for d in defs:
            if d["name"] in seen:
                raise ValueError(f"counter {d['name']!r} is defined twice")
            seen.add(d["name"])
            self.defs.append({**d, "ast": parse(str(d["expression"]))})

    @staticmethod
    def load(path: Optional[str] = None) -> "CounterSet":
        import yaml

        p = Path(path) if path else Path(__file__).with_name("counter_defs.yaml")
        return CounterSet(yaml.safe_load(p.read_text())["counters"])

    def required_metrics(self) -> List[str]:
        """Raw metric names the definitions read (what to pass to ``ncu --metrics``)."""
        names = sorted({i for d in self.defs for i in identifiers(d["ast"]) if not i.startswith(("peak.", "arg."))})
        return names

    def evaluate(self, raw: Dict[str, float], peaks: Optional[dict] = None, args: Optional[dict] = None) -> Dict[str, Optional[float]]:
        env = dict(raw)
        env.update({f"peak.{k}": v for k, v in (peaks or {}).items() if isinstance(v, (int, float))})
        env.update({f"arg.{k}": v for k, v in (args or {}).items()})
        out: Dict[str, Optional[float]] = {}
        for d in self.defs:
            try:
                out[d["name"]] = evaluate(d["ast"], env)
            except KeyError:
                out[d["name"]] = None  # an input is not in this capture
        return out


def collect_command(metrics: Sequence[str], command: Sequence[str], kernel: str, count: int, skip: int, output: str) -> List[str]:
    """The Nsight Compute line that gathers ``metrics`` for ``count`` launches of kernels matching ``kernel``."""
    cmd = ["ncu", "--clock-control", "none", "--metrics", ",".join(metrics), "-c", str(int(count)), "-o", output, "-f"]
    if kernel:
        cmd += ["-k", f"regex:{kernel}"]
    if skip:
        cmd += ["-s", str(int(skip))]
    return cmd + list(command)


PANELS = ["speed_of_light", "memory", "cache", "compute", "occupancy", "launch"]
_STALL = re.compile(r"^smsp__average_warps_issue_stalled_(.+)_per_issue_active\.ratio$")
_STALL_HINT = {
    "long_scoreboard": "waiting for global / local memory (or a remote rank's memory)",
    "short_scoreboard": "waiting for shared memory or special-function results",
    "barrier": "waiting at a CTA barrier",
    "membar": "waiting for a memory fence",
    "wait": "fixed-latency dependency",
    "lg_throttle": "load/store queue full (too many memory instructions in flight per warp)",
    "math_pipe_throttle": "the pipe the warp needs is busy",
    "mio_throttle": "shared-memory / special-function queue full",
    "tex_throttle": "texture / L1 queue full",
    "not_selected": "eligible, another warp was issued (enough parallelism)",
    "no_instruction": "instruction fetch",
    "dispatch_stall": "dispatch unit busy",
    "sleeping": "in nanosleep (a polling loop backing off)",
    "drain": "draining stores at exit",
    "imc_miss": "constant cache miss",
    "branch_resolving": "waiting for a branch target",
    "selected": "issuing",
}


def stall_ranking(raw: Dict[str, float], top: int = 5) -> List[Tuple[str, float, str]]:
    """The warp stall reasons of a capture, largest first: (reason, stalled warps per issued instruction, what it means)."""
    found = []
    for name, v in raw.items():
        m = _STALL.match(name)
        if m and m.group(1) != "selected" and v == v:
            found.append((m.group(1), float(v), _STALL_HINT.get(m.group(1), "")))
    found.sort(key=lambda t: -t[1])
    return found[:top]


def verdict(values: Dict[str, Optional[float]], stalls: Sequence[Tuple[str, float, str]]) -> str:
    """One line on what bounds the launch, from the speed-of-light counters (the analysis front page of the reference's
    rocprofiler-compute, restated on these counters)."""
    g = lambda k: values.get(k) if values.get(k) is not None else 0.0  # noqa: E731
    mem = max(g("hbm_fraction") * 100, g("dram_throughput_pct"), g("memory_throughput_pct"))
    frac = values.get("bf16_fraction") or 0.0
    cmp_ = max(g("tensor_active_pct"), g("sm_throughput_pct"), frac * 100 if frac <= 1.2 else 0.0)   # arg.flops of another kernel gives nonsense
    if mem >= 60 and mem >= cmp_:
        return f"memory bound ({mem:.0f} % of the memory system's peak)"
    if cmp_ >= 60:
        return f"compute bound ({cmp_:.0f} % of the busiest SM unit)"
    why = f"; warps mostly stall on {stalls[0][0]} ({stalls[0][2]})" if stalls else ""
    if g("sm_active_pct") and g("sm_active_pct") < 50:
        return f"under-filled: SMs had work in {g('sm_active_pct'):.0f} % of the cycles (grid of {g('grid_size'):.0f} CTAs, {g('waves_per_sm'):.2f} waves){why}"
    return f"latency bound: memory {mem:.0f} %, compute {cmp_:.0f} % of peak{why}"


def analyze(cs: "CounterSet", kernels, peaks: dict, args: dict) -> List[dict]:
    """Per captured launch: the derived counters grouped by panel, the stall ranking and the verdict."""
    out = []
    for k in kernels:
        raw = dict(k.raw) if hasattr(k, "raw") else {}
        values = cs.evaluate(raw, peaks, args)
        panels: Dict[str, list] = {p: [] for p in PANELS}
        for d in cs.defs:
            v = values.get(d["name"])
            if v is not None and v == v:
                panels.setdefault(d.get("panel", "speed_of_light"), []).append({"name": d["name"], "value": v, "unit": d.get("unit", ""), "description": d.get("description", "")})
        stalls = stall_ranking(raw)
        out.append({"kernel": k.name, "panels": {p: rows for p, rows in panels.items() if rows},
                    "stalls": [{"reason": r, "warps_per_issue": v, "meaning": h} for r, v, h in stalls], "verdict": verdict(values, stalls)})
    return out


def compare(cs: "CounterSet", base, other, peaks: dict, args: dict) -> List[dict]:
    """Two captures of the same program side by side (the reference's analyze mode with a baseline path): launches are
    paired by kernel name in order of appearance (the i-th launch of a name in one capture with the i-th in the other);
    every counter both could evaluate is listed with its value in each and the relative change."""
    def by_name(kernels):
        seen: Dict[str, int] = {}
        out = {}
        for k in kernels:
            i = seen.get(k.name, 0)
            seen[k.name] = i + 1
            out[(k.name, i)] = k
        return out

    a, b = by_name(base), by_name(other)
    rows = []
    for key in a:
        if key not in b:
            continue
        va, vb = cs.evaluate(dict(a[key].raw), peaks, args), cs.evaluate(dict(b[key].raw), peaks, args)
        counters_ = []
        for d in cs.defs:
            x, y = va.get(d["name"]), vb.get(d["name"])
            if x is None or y is None or x != x or y != y:
                continue
            counters_.append({"name": d["name"], "unit": d.get("unit", ""), "base": x, "other": y, "change_pct": (y - x) / abs(x) * 100 if x else None})
        rows.append({"kernel": key[0], "launch": key[1], "counters": counters_})
    return rows


def format_comparison(rows: Sequence[dict], threshold_pct: float = 0.0) -> str:
    lines = []
    for r in rows:
        lines.append(f"== {r['kernel']} (launch {r['launch']})")
        for c in r["counters"]:
            ch = c["change_pct"]
            if ch is not None and abs(ch) < threshold_pct:
                continue
            lines.append(f"     {c['name']:<30} {c['base']:>12.4g} -> {c['other']:>12.4g} {c['unit']:<24} {'' if ch is None else f'{ch:+.1f} %'}")
    return "\n".join(lines)


def format_analysis(items: Sequence[dict]) -> str:
    lines = []
    for it in items:
        lines.append(f"== {it['kernel']}")
        lines.append(f"   {it['verdict']}")
        for p, rows in it["panels"].items():
            lines.append(f"   [{p}]")
            for r in rows:
                lines.append(f"     {r['name']:<30} {r['value']:>12.4g} {r['unit']:<28} {r['description']}")
        if it["stalls"]:
            lines.append("   [stalls: stalled warps per issued instruction]")
            for s_ in it["stalls"]:
                lines.append(f"     {s_['reason']:<30} {s_['warps_per_issue']:>12.3g} {'':<28} {s_['meaning']}")
    return "\n".join(lines)


def html_report(items: Sequence[dict], title: str = "Kernel analysis") -> str:
    """The analysis as one self-contained HTML page (no scripts, no external files): per launch the verdict, one table per
    panel with a bar for every percentage, and the stall ranking as bars. The reference offers its analysis in a browser
    too (rocprofiler-compute src/rocprof_compute_analyze/analysis_webui.py); this is the static counterpart."""
    import html

    def esc(x) -> str:
        return html.escape(str(x))

    def bar(frac: float, color: str) -> str:
        w = max(0.0, min(1.0, frac)) * 100.0
        return f'<div class="bar"><div style="width:{w:.1f}%;background:{color}"></div></div>'

    out = ["<!doctype html><html><head><meta charset='utf-8'>", f"<title>{esc(title)}</title>",
           "<style>body{font:14px/1.4 system-ui,sans-serif;margin:2em;max-width:1100px}h2{margin-top:2em;font-size:16px;word-break:break-all}"
           "table{border-collapse:collapse;width:100%;margin:.4em 0 1em}td,th{padding:2px 8px;text-align:left;border-bottom:1px solid #ddd;vertical-align:top}"
           "td.n{text-align:right;font-variant-numeric:tabular-nums;white-space:nowrap}.bar{width:160px;height:10px;background:#eee;border-radius:2px}"
           ".bar div{height:10px;border-radius:2px}.verdict{background:#f4f4f4;padding:.5em .8em;border-left:4px solid #888}h3{font-size:13px;margin:.8em 0 .2em;"
           "text-transform:uppercase;color:#555}nav a{display:block;word-break:break-all}</style></head><body>", f"<h1>{esc(title)}</h1>", "<nav>"]
    for i, it in enumerate(items):
        out.append(f'<a href="#k{i}">{i}. {esc(it["kernel"][:140])}</a>')
    out.append("</nav>")
    for i, it in enumerate(items):
        out.append(f'<h2 id="k{i}">{i}. {esc(it["kernel"])}</h2><p class="verdict">{esc(it["verdict"])}</p>')
        for panel, rows in it["panels"].items():
            out.append(f"<h3>{esc(panel.replace('_', ' '))}</h3><table><tr><th>counter</th><th>value</th><th>unit</th><th></th><th>meaning</th></tr>")
            for r in rows:
                pct = "%" in r["unit"] or "percent" in r["unit"]
                cell = bar(r["value"] / 100.0, "#4a90d9" if r["value"] < 80 else "#d9534f") if pct else ""
                out.append(f'<tr><td>{esc(r["name"])}</td><td class="n">{r["value"]:.4g}</td><td>{esc(r["unit"])}</td><td>{cell}</td><td>{esc(r["description"])}</td></tr>')
            out.append("</table>")
        if it["stalls"]:
            top = max(s_["warps_per_issue"] for s_ in it["stalls"]) or 1.0
            out.append("<h3>stalls (stalled warps per issued instruction)</h3><table><tr><th>reason</th><th>value</th><th></th><th>meaning</th></tr>")
            for s_ in it["stalls"]:
                out.append(f'<tr><td>{esc(s_["reason"])}</td><td class="n">{s_["warps_per_issue"]:.3g}</td><td>{bar(s_["warps_per_issue"] / top, "#e0a030")}</td>'
                           f'<td>{esc(s_["meaning"])}</td></tr>')
            out.append("</table>")
    out.append("</body></html>")
    return "\n".join(out)


def main(argv: Optional[Sequence[str]] = None) -> int:
    from . import roofline

    ap = argparse.ArgumentParser(prog="counters", description=__doc__.split("\n\n")[0])
    ap.add_argument("inputs", nargs="*", help=".ncu-rep files or raw-page CSV files")
    ap.add_argument("--defs", default=None, help="YAML definitions (default: the file next to this module)")
    ap.add_argument("--peaks", default="MEASURED_PEAKS.json")
    ap.add_argument("--arg", action="append", default=[], help="NAME=VALUE readable as arg.NAME")
    ap.add_argument("--list", action="store_true", help="print the definitions and the raw metrics they need")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--list-kernels", action="store_true", help="the kernels of the capture(s) with how often each was captured and its total time, and stop "
                    "(names to give --kernel-filter)")
    ap.add_argument("--compare", default="", metavar="OTHER", help="a second report or CSV of the same program: counters of matching launches side by side with the change")
    ap.add_argument("--min-change", type=float, default=0.0, metavar="PCT", help="with --compare: only counters that changed by at least this much")
    ap.add_argument("--kernel-filter", default="", metavar="REGEX", help="with --analyze / --compare: only launches whose kernel name matches")
    ap.add_argument("--analyze", action="store_true", help="per launch: the counters grouped by panel (speed of light, memory, caches, compute, "
                    "occupancy, launch), the warp stall ranking and a one-line verdict on what bounds it")
    ap.add_argument("--html", default="", metavar="FILE", help="with --analyze: write the analysis as one self-contained HTML page as well")
    ap.add_argument("--collect", action="store_true", help="run the command after -- under Nsight Compute for the metrics the counters need, then evaluate")
    ap.add_argument("--counter", action="append", default=[], help="with --collect: only these definitions (default: all)")
    ap.add_argument("-k", "--kernel", default="", help="with --collect: regular expression of the kernels to capture")
    ap.add_argument("-c", "--count", type=int, default=3, help="with --collect: launches to capture (kept small on purpose)")
    ap.add_argument("-s", "--skip", type=int, default=0, help="with --collect: matching launches to skip first")
    ap.add_argument("-o", "--output", default="counters_capture", help="with --collect: report file (without .ncu-rep)")
    ap.add_argument("--print-command", action="store_true", help="with --collect: print the ncu line and stop")
    argv = list(sys.argv[1:] if argv is None else argv)
    command: List[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, command = argv[:i], argv[i + 1:]
    a = ap.parse_args(argv)
    cs = CounterSet.load(a.defs)
    if a.collect:
        import subprocess

        if not command:
            ap.error("--collect needs a command after --")
        if a.count < 1 or a.count > 20:
            ap.error("--count must be between 1 and 20: a capture replays every launch many times")
        if a.counter:
            known = {d["name"] for d in cs.defs}
            missing = [c for c in a.counter if c not in known]
            if missing:
                ap.error(f"unknown counter(s): {', '.join(missing)}")
            cs = CounterSet([d for d in cs.defs if d["name"] in a.counter])
        cmd = collect_command(cs.required_metrics(), command, a.kernel, a.count, a.skip, a.output)
        if a.print_command:
            print(" ".join(cmd))
            return 0
        rc = subprocess.call(cmd)
        if rc != 0:
            print(f"counters: ncu exited with {rc}", file=sys.stderr)
            return rc
        a.inputs = [a.output + ".ncu-rep"]
        try:   # the machine the capture was taken on, beside it (the reference keeps a sysinfo file with every profiled workload)
            from . import info

            with open(a.output + "_sysinfo.json", "w") as f:
                json.dump({"host": info.host_info(), "devices": info.device_info(), "library": info.library_info(), "command": command,
                           "counters": [d["name"] for d in cs.defs]}, f, indent=1)
        except Exception as e:  # noqa: BLE001  a note beside the capture must not fail the capture
            print(f"counters: no sysinfo file ({type(e).__name__}: {e})", file=sys.stderr)
    if a.list:
        for d in cs.defs:
            print(f"{d['name']:<22} [{d.get('unit', '')}] = {d['expression']}\n{'':<22} {d.get('description', '')}")
        print("\nraw metrics: " + ",".join(cs.required_metrics()))
        return 0
    if a.list_kernels:
        seen: Dict[str, list] = {}
        for path in a.inputs:
            for k in roofline.read_ncu(path):
                raw = dict(k.raw) if hasattr(k, "raw") else {}
                e = seen.setdefault(k.name, [0, 0.0])
                e[0] += 1
                e[1] += float(raw.get("gpu__time_duration.sum", 0.0) or 0.0)
        rows_ = [{"kernel": n, "launches": c, "total_us": t / 1e3} for n, (c, t) in sorted(seen.items(), key=lambda kv: -kv[1][1])]
        if a.json:
            print(json.dumps(rows_, indent=1))
        else:
            for r in rows_:
                print(f"{r['launches']:>5} x {r['total_us']:>12.1f} us  {r['kernel']}")
        return 0
    peaks = roofline.load_peaks(a.peaks)
    args = {k: float(v) for k, v in (s.split("=", 1) for s in a.arg)}
    rows = []
    for path in a.inputs:
        for k in roofline.read_ncu(path):
            raw = dict(k.raw) if hasattr(k, "raw") else {}
            rows.append({"kernel": k.name, **cs.evaluate(raw, peaks, args)})
    keep = (lambda ks: [k for k in ks if re.search(a.kernel_filter, k.name)]) if a.kernel_filter else (lambda ks: list(ks))
    if a.compare:
        if len(a.inputs) != 1:
            ap.error("--compare takes exactly one input to compare OTHER with")
        rows_ = compare(cs, keep(roofline.read_ncu(a.inputs[0])), keep(roofline.read_ncu(a.compare)), peaks, args)
        print(json.dumps(rows_, indent=1) if a.json else format_comparison(rows_, a.min_change))
        return 0
    if a.analyze:
        items = [it for path in a.inputs for it in analyze(cs, keep(roofline.read_ncu(path)), peaks, args)]
        if a.html:
            with open(a.html, "w") as f:
                f.write(html_report(items, "Kernel analysis: " + ", ".join(os.path.basename(p) for p in a.inputs)))
        print(json.dumps(items, indent=1) if a.json else format_analysis(items))
        return 0
    if a.json:
        print(json.dumps(rows, indent=1))
    else:
        for r in rows:
            print(r["kernel"])
            for name, v in r.items():
                if name != "kernel" and v is not None:
                    print(f"  {name:<22} {v:.4g}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
