"""Static resource report of every kernel in the library: registers per thread, shared memory,
stack frame and spills, as the assembler reports them (``nvcc -Xptxas -v``). No GPU needed.

    python -m rocm_systems_b200.utils.ptxas_report [-o report.md]

Kernel names are demangled with ``c++filt`` when it is available.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import re
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path
from typing import List, Optional, Sequence

from . import build

ENTRY = re.compile(r"Compiling entry function '([^']+)' for 'sm_100a'")
PROPS = re.compile(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads")
USED = re.compile(r"Used (\d+) registers(?:, used (\d+) barriers)?(?:, (\d+) bytes cumulative stack size)?(?:, (\d+) bytes smem)?")


def parse(text: str) -> List[dict]:
    out, cur = [], None
    for line in text.splitlines():
        m = ENTRY.search(line)
        if m:
            cur = {"mangled": m.group(1), "stack": 0, "spill_stores": 0, "spill_loads": 0, "registers": 0, "smem": 0}
            out.append(cur)
            continue
        if cur is None:
            continue
        m = PROPS.search(line)
        if m:
            cur["stack"], cur["spill_stores"], cur["spill_loads"] = map(int, m.groups())
        m = USED.search(line)
        if m:
            cur["registers"] = int(m.group(1))
            sm = re.search(r"(\d+) bytes smem", line)
            cur["smem"] = int(sm.group(1)) if sm else 0
    return out


def demangle(names: Sequence[str]) -> List[str]:
    if not names or shutil.which("c++filt") is None:
        return list(names)
    p = subprocess.run(["c++filt"], input="\n".join(names), capture_output=True, text=True)
    res = p.stdout.splitlines()
    return res if len(res) == len(names) else list(names)


def short(name: str) -> str:
    name = re.sub(r"\(anonymous namespace\)::", "", name)
    name = re.sub(r"\(.*$", "", name)           # drop the parameter list
    name = name.replace("b200::", "")
    return name if len(name) <= 110 else name[:107] + "..."


def collect() -> List[dict]:
    jobs = [(src, defs) for src, _, defs in build.lib_jobs() if src.suffix == ".cu"]
    rows: List[dict] = []
    with tempfile.TemporaryDirectory() as d:
        def one(job):
            src, defs = job
            tag = "_".join(x.replace("-D", "").replace("=", "") for x in defs) or "x"
            cmd = [build.NVCC, *build.ARCH, *build.COMMON, *defs, "-Xptxas", "-v", "-c", str(src), "-o", str(Path(d) / f"{src.stem}_{tag[:40]}.o")]
            p = subprocess.run(cmd, capture_output=True, text=True)
            if p.returncode != 0:
                raise RuntimeError(p.stderr[-2000:])
            ks = parse(p.stderr + p.stdout)
            for k in ks:
                k["file"] = str(src.relative_to(build.CSRC))
            return ks
        with cf.ThreadPoolExecutor(max_workers=8) as ex:
            for ks in ex.map(one, jobs):
                rows += ks
    names = demangle([r["mangled"] for r in rows])
    for r, n in zip(rows, names):
        r["name"] = short(n)
    return rows


def render(rows: List[dict]) -> str:
    lines = ["| file | kernel | registers | static smem (B) | stack (B) | spill st/ld (B) |", "|---|---|---|---|---|---|"]
    seen = set()
    for r in sorted(rows, key=lambda r: (r["file"], r["name"])):
        key = (r["file"], r["name"], r["registers"], r["smem"], r["stack"], r["spill_stores"])
        if key in seen:
            continue
        seen.add(key)
        lines.append(f"| {r['file']} | `{r['name']}` | {r['registers']} | {r['smem']} | {r['stack']} | {r['spill_stores']}/{r['spill_loads']} |")
    return "\n".join(lines) + "\n"


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("-o", "--output", default="")
    a = ap.parse_args(argv)
    text = render(collect())
    if a.output:
        Path(a.output).write_text(text)
    else:
        sys.stdout.write(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
