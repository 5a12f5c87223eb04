"""Roofline and speed-of-light report for kernels, from Nsight Compute counters or from plain timings.

The counterpart of the reference's ``rocprof-compute`` analyze mode (rocprofiler-compute/src:
``rocprof_compute_analyze``, the speed-of-light and memory-chart panels, ``roofline.py``): for each
kernel, where it sits against the device's measured ceilings and which of them bounds it.

Inputs
  * an ``.ncu-rep`` file (read through ``ncu -i FILE --page raw --csv``) or that CSV itself, or
  * ``--point NAME:FLOPS:BYTES:SECONDS`` for kernels timed with events (algorithmic work).
Ceilings come from a JSON file with ``hbm_gbs`` and ``bf16_tflops`` (a measured copy bandwidth and
a measured library GEMM rate); without one the nominal B200 figures are used and labelled so.

    python -m rocm_systems_b200.tools.roofline prof.ncu-rep --peaks MEASURED_PEAKS.json
    python -m rocm_systems_b200.tools.roofline --point gemm8k:1.0995e12:4.03e8:7.15e-4 --plot
"""
from __future__ import annotations

import argparse
import csv
import io
import json
import math
import subprocess
import sys
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Sequence

NOMINAL = {"hbm_gbs": 7700.0, "bf16_tflops": 2250.0, "source": "nominal"}

# raw-page metric -> short key
METRICS = {
    "gpu__time_duration.sum": "duration_ns",
    "dram__bytes_read.sum": "dram_read_bytes",
    "dram__bytes_write.sum": "dram_write_bytes",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed": "dram_pct",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active": "tensor_pct",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed": "sm_pct",
    "sm__warps_active.avg.pct_of_peak_sustained_active": "occupancy_pct",
    "launch__registers_per_thread": "registers",
    "launch__grid_size": "grid",
    "launch__block_size": "block",
    "lts__t_sector_hit_rate.pct": "l2_hit_pct",
    "smsp__cycles_active.avg": "active_cycles",
}
UNIT_SCALE = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12, "ns": 1.0, "us": 1e3, "usecond": 1e3, "ms": 1e6, "msecond": 1e6,
              "nsecond": 1.0, "second": 1e9, "s": 1e9}


@dataclass
class Kernel:
    name: str
    duration_ns: float = 0.0
    dram_bytes: float = 0.0
    flops: float = 0.0          # algorithmic, when known
    counters: Dict[str, float] = field(default_factory=dict)
    raw: Dict[str, float] = field(default_factory=dict)   # every numeric column of the report under its raw name

    @property
    def gbs(self) -> float:
        return self.dram_bytes / self.duration_ns if self.duration_ns else 0.0

    @property
    def tflops(self) -> float:
        return self.flops / self.duration_ns / 1e3 if self.duration_ns else 0.0

    @property
    def intensity(self) -> float:
        return self.flops / self.dram_bytes if self.dram_bytes else 0.0


def load_peaks(path: Optional[str]) -> dict:
    if path and Path(path).exists():
        d = json.loads(Path(path).read_text())
        out = {"hbm_gbs": float(d.get("hbm_gbs", NOMINAL["hbm_gbs"])), "bf16_tflops": float(d.get("bf16_tflops", NOMINAL["bf16_tflops"])),
               "source": "measured"}
        if "bf16_tflops_sustained" in d:
            out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
        return out
    return dict(NOMINAL)


def parse_ncu_csv(text: str) -> List[Kernel]:
    """Parses ``ncu --page raw --csv`` output: a header row, a units row, then one row per launch."""
    lines = [l for l in text.splitlines() if l.startswith('"')]
    rows = list(csv.reader(io.StringIO("\n".join(lines))))
    if len(rows) < 3:
        return []
    header, units = rows[0], rows[1]
    col = {n: i for i, n in enumerate(header)}
    name_col = col.get("Kernel Name", col.get("Function Name"))
    out = []
    for r in rows[2:]:
        if name_col is None or len(r) <= name_col:
            continue
        k = Kernel(name=r[name_col])
        for metric, key in METRICS.items():
            i = col.get(metric)
            if i is None or i >= len(r) or r[i] in ("", "n/a"):
                continue
            try:
                v = float(r[i].replace(",", ""))
            except ValueError:
                continue
            k.counters[key] = v * UNIT_SCALE.get(units[i], 1.0) if key.endswith(("_bytes", "_ns")) else v
        # every numeric column under its raw name, bytes and times normalised (for tools/counters.py)
        for name, i in col.items():
            if i < len(r) and r[i] not in ("", "n/a"):
                try:
                    k.raw[name] = float(r[i].replace(",", "")) * UNIT_SCALE.get(units[i], 1.0)
                except ValueError:
                    pass
        k.duration_ns = k.counters.get("duration_ns", 0.0)
        k.dram_bytes = k.counters.get("dram_read_bytes", 0.0) + k.counters.get("dram_write_bytes", 0.0)
        out.append(k)
    return out


def read_ncu(path: str) -> List[Kernel]:
    if path.endswith(".ncu-rep"):
        text = subprocess.run(["ncu", "-i", path, "--page", "raw", "--csv"], capture_output=True, text=True, check=True).stdout
    else:
        text = Path(path).read_text()
    return parse_ncu_csv(text)


def classify(k: Kernel, peaks: dict) -> str:
    """Which ceiling bounds the kernel: the nearer of the two, or latency when both are far."""
    mem = k.gbs / peaks["hbm_gbs"] if peaks["hbm_gbs"] else 0.0
    cmp_ = k.tflops / peaks["bf16_tflops"] if k.flops else k.counters.get("tensor_pct", 0.0) / 100.0
    if max(mem, cmp_) < 0.3:
        return "latency/occupancy"
    return "memory" if mem >= cmp_ else "compute"


def report(kernels: Sequence[Kernel], peaks: dict) -> str:
    label = "of measured" if peaks["source"] == "measured" else "of nominal"
    head = ["kernel", "time_us", "DRAM_MB", "GB/s", f"HBM_frac({label})", "TFLOP/s", f"bf16_frac({label})", "tensor%", "occ%", "regs", "bound"]
    rows = []
    for k in kernels:
        c = k.counters
        rows.append([k.name[:48], f"{k.duration_ns / 1e3:.1f}", f"{k.dram_bytes / 1e6:.1f}", f"{k.gbs:.0f}", f"{k.gbs / peaks['hbm_gbs']:.2f}",
                     f"{k.tflops:.0f}" if k.flops else "-", f"{k.tflops / peaks['bf16_tflops']:.2f}" if k.flops else "-",
                     f"{c['tensor_pct']:.0f}" if "tensor_pct" in c else "-", f"{c['occupancy_pct']:.0f}" if "occupancy_pct" in c else "-",
                     f"{c['registers']:.0f}" if "registers" in c else "-", classify(k, peaks)])
    widths = [max(len(str(r[i])) for r in [head] + rows) for i in range(len(head))]
    fmt = lambda r: "  ".join(str(c).ljust(w) for c, w in zip(r, widths))  # noqa: E731
    lines = [f"ceilings ({peaks['source']}): HBM {peaks['hbm_gbs']:.0f} GB/s, bf16 {peaks['bf16_tflops']:.0f} TFLOP/s"
             f" (ridge at {peaks['bf16_tflops'] * 1e3 / peaks['hbm_gbs']:.0f} FLOP/byte)", fmt(head), fmt(["-" * w for w in widths])]
    lines += [fmt(r) for r in rows]
    return "\n".join(lines)


def ascii_plot(kernels: Sequence[Kernel], peaks: dict, width: int = 72, height: int = 20) -> str:
    """log-log roofline: x arithmetic intensity (FLOP/byte), y TFLOP/s; '/' and '-' draw the roof."""
    pts = [(k.intensity, k.tflops, k.name) for k in kernels if k.flops and k.dram_bytes]
    x0, x1 = -1.0, 5.0                       # 0.1 .. 100000 FLOP/byte
    y1 = math.log10(peaks["bf16_tflops"] * 2)
    y0 = y1 - 4.0
    grid = [[" "] * width for _ in range(height)]

    def cell(x: float, y: float):
        cx = int((math.log10(max(x, 1e-9)) - x0) / (x1 - x0) * (width - 1))
        cy = int((y1 - math.log10(max(y, 1e-9))) / (y1 - y0) * (height - 1))
        return cx, cy

    for cx in range(width):
        x = 10 ** (x0 + (x1 - x0) * cx / (width - 1))
        roof = min(peaks["bf16_tflops"], x * peaks["hbm_gbs"] / 1e3)
        _, cy = cell(x, roof)
        if 0 <= cy < height:
            grid[cy][cx] = "-" if roof >= peaks["bf16_tflops"] else "/"
    legend = []
    for i, (x, y, name) in enumerate(pts):
        cx, cy = cell(x, y)
        mark = chr(ord("A") + i % 26)
        if 0 <= cx < width and 0 <= cy < height:
            grid[cy][cx] = mark
        legend.append(f"  {mark}: {name[:50]}  {x:.1f} FLOP/B  {y:.0f} TFLOP/s")
    out = ["TFLOP/s (log)"] + ["|" + "".join(r) for r in grid] + ["+" + "-" * width, " " * 20 + "arithmetic intensity, FLOP/byte (log, 0.1 .. 1e5)"]
    return "\n".join(out + legend)


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="roofline", description=__doc__.split("\n\n")[0])
    ap.add_argument("inputs", nargs="*", help=".ncu-rep files or raw-page CSV files")
    ap.add_argument("--peaks", default="MEASURED_PEAKS.json")
    ap.add_argument("--point", action="append", default=[], help="NAME:FLOPS:BYTES:SECONDS (algorithmic work and an event timing)")
    ap.add_argument("--flops", action="append", default=[], help="REGEX=FLOPS: algorithmic FLOPs per launch for kernels whose name matches")
    ap.add_argument("--plot", action="store_true")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    peaks = load_peaks(a.peaks)
    kernels: List[Kernel] = []
    for p in a.inputs:
        kernels += read_ncu(p)
    import re

    for spec in a.flops:
        rx, val = spec.rsplit("=", 1)
        for k in kernels:
            if re.search(rx, k.name):
                k.flops = float(val)
    for spec in a.point:
        name, fl, by, sec = spec.rsplit(":", 3)
        kernels.append(Kernel(name=name, duration_ns=float(sec) * 1e9, dram_bytes=float(by), flops=float(fl)))
    if not kernels:
        ap.error("nothing to report: give an ncu report/CSV or --point")
    if a.json:
        print(json.dumps({"peaks": peaks, "kernels": [{"name": k.name, "duration_ns": k.duration_ns, "dram_bytes": k.dram_bytes, "gbs": k.gbs,
                                                       "tflops": k.tflops, "hbm_fraction": k.gbs / peaks["hbm_gbs"],
                                                       "bf16_fraction": k.tflops / peaks["bf16_tflops"], "bound": classify(k, peaks),
                                                       "counters": k.counters} for k in kernels]}, indent=1))
    else:
        print(report(kernels, peaks))
        if a.plot:
            print()
            print(ascii_plot(kernels, peaks))
    return 0


if __name__ == "__main__":
    sys.exit(main())
