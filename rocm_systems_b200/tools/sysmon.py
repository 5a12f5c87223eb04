"""Background system sampler: GPU readings (through NVML), host CPU utilisation, frequency, load and memory, and per chosen
process its resident set, CPU utilisation, thread count, page faults and context switches, on the same clock as the tracers,
written as counter tracks.

The counterpart of the reference's process sampler in its system profiler (rocprofiler-systems:
background thread reading amd-smi, CPU frequency and memory while the application runs, shown as
Perfetto counter tracks). The tracing launcher starts it with ``--sys-sample PERIOD_MS``.

    with SystemSampler(period_ms=100, pids=[child.pid]) as s: child.wait()
    s.write_csv("run.sysmon.csv")
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional, Sequence, Tuple

GPU_FIELDS = ("sm_clock", "power", "temp", "gpu_util", "mem_used")


def _cpu_times() -> Tuple[int, int]:
    with open("/proc/stat") as f:
        parts = f.readline().split()[1:]
    vals = list(map(int, parts))
    idle = vals[3] + (vals[4] if len(vals) > 4 else 0)
    return sum(vals), idle


def _meminfo() -> Dict[str, int]:
    out = {}
    with open("/proc/meminfo") as f:
        for line in f:
            k, v = line.split(":", 1)
            if k in ("MemTotal", "MemAvailable"):
                out[k] = int(v.split()[0]) * 1024
    return out


def _rss(pid: int) -> Optional[int]:
    try:
        with open(f"/proc/{pid}/status") as f:
            for line in f:
                if line.startswith("VmRSS:"):
                    return int(line.split()[1]) * 1024
    except OSError:
        return None
    return None


def _cpu_freq_mhz() -> Optional[float]:
    """Mean current frequency of the host CPUs (cpufreq when the kernel exposes it, else the `cpu MHz` lines of /proc/cpuinfo)."""
    import glob

    vals = []
    for path in glob.glob("/sys/devices/system/cpu/cpu[0-9]*/cpufreq/scaling_cur_freq"):
        try:
            with open(path) as f:
                vals.append(int(f.read()) / 1000.0)
        except (OSError, ValueError):
            pass
    if not vals:
        try:
            with open("/proc/cpuinfo") as f:
                vals = [float(line.split(":")[1]) for line in f if line.lower().startswith("cpu mhz")]
        except (OSError, ValueError):
            vals = []
    return sum(vals) / len(vals) if vals else None


def _loadavg() -> Optional[float]:
    try:
        with open("/proc/loadavg") as f:
            return float(f.read().split()[0])
    except (OSError, ValueError):
        return None


def _proc_stat(pid: int) -> Optional[Dict[str, int]]:
    """CPU ticks (user + system), page faults and thread count of a process from /proc/<pid>/stat."""
    try:
        with open(f"/proc/{pid}/stat") as f:
            text = f.read()
    except OSError:
        return None
    rest = text[text.rfind(")") + 2:].split()     # the command may contain spaces and parentheses: fields start behind the last ')'
    try:
        return {"minflt": int(rest[7]), "majflt": int(rest[9]), "ticks": int(rest[11]) + int(rest[12]), "threads": int(rest[17])}
    except (IndexError, ValueError):
        return None


def _proc_ctx_switches(pid: int) -> Optional[Tuple[int, int]]:
    try:
        vol = invol = None
        with open(f"/proc/{pid}/status") as f:
            for line in f:
                if line.startswith("voluntary_ctxt_switches:"):
                    vol = int(line.split()[1])
                elif line.startswith("nonvoluntary_ctxt_switches:"):
                    invol = int(line.split()[1])
        return (vol, invol) if vol is not None and invol is not None else None
    except (OSError, ValueError):
        return None


class SystemSampler:
    """Background thread that samples GPU readings (NVML) and host counters at a fixed period; a context manager."""

    def __init__(self, period_ms: int = 100, pids: Sequence[int] = (), gpu: bool = True, gpu_fields: Sequence[str] = GPU_FIELDS):
        self.period = period_ms / 1e3
        self.pids = list(pids)
        self.samples: List[Tuple[str, int, int, float]] = []  # (counter, device or pid, monotonic ns, value)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.gpu_fields = list(gpu_fields)
        self._last_proc: Dict[int, Tuple[int, int]] = {}   # pid -> (monotonic ns, cpu ticks) of the previous sample
        self.smi = None
        self.ngpu = 0
        if gpu:
            try:
                from .smi import Smi

                self.smi = Smi()
                self.ngpu = self.smi.count()
            except Exception:  # noqa: BLE001 - no NVML here: host counters only
                self.smi = None

    def sample_once(self) -> None:
        now = time.monotonic_ns()
        total, idle = _cpu_times()
        if self._last_cpu is not None:
            dt, di = total - self._last_cpu[0], idle - self._last_cpu[1]
            if dt > 0:
                self.samples.append(("host_cpu_util_percent", -1, now, 100.0 * (dt - di) / dt))
        self._last_cpu = (total, idle)
        mem = _meminfo()
        if mem:
            self.samples.append(("host_mem_used_bytes", -1, now, float(mem.get("MemTotal", 0) - mem.get("MemAvailable", 0))))
        freq = _cpu_freq_mhz()
        if freq is not None:
            self.samples.append(("host_cpu_freq_mhz", -1, now, freq))
        load = _loadavg()
        if load is not None:
            self.samples.append(("host_load_1min", -1, now, load))
        for pid in self.pids:
            r = _rss(pid)
            if r is not None:
                self.samples.append(("process_rss_bytes", pid, now, float(r)))
            st = _proc_stat(pid)
            if st is not None:
                self.samples.append(("process_threads", pid, now, float(st["threads"])))
                self.samples.append(("process_page_faults_minor", pid, now, float(st["minflt"])))
                self.samples.append(("process_page_faults_major", pid, now, float(st["majflt"])))
                last = self._last_proc.get(pid)
                if last is not None and now > last[0]:
                    import os

                    hz = os.sysconf("SC_CLK_TCK") or 100
                    self.samples.append(("process_cpu_util_percent", pid, now, 100.0 * (st["ticks"] - last[1]) / hz / ((now - last[0]) / 1e9)))
                self._last_proc[pid] = (now, st["ticks"])
            cs = _proc_ctx_switches(pid)
            if cs is not None:
                self.samples.append(("process_ctx_switches_voluntary", pid, now, float(cs[0])))
                self.samples.append(("process_ctx_switches_involuntary", pid, now, float(cs[1])))
        if self.smi is not None:
            for d in range(self.ngpu):
                for f in self.gpu_fields:
                    try:
                        self.samples.append((f"gpu_{f}", d, now, float(self.smi.read(d, f))))
                    except RuntimeError:
                        pass

    _last_cpu: Optional[Tuple[int, int]] = None

    def _run(self) -> None:
        while not self._stop.wait(self.period):
            self.sample_once()

    def start(self) -> "SystemSampler":
        self.sample_once()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.period * 2 + 1)
        self.sample_once()

    __enter__ = start

    def __exit__(self, *exc) -> None:
        self.stop()

    def write_csv(self, path: str) -> int:
        with open(path, "w") as f:
            f.write('"Counter","Device","Timestamp","Value"\n')
            for name, dev, ts, val in self.samples:
                f.write(f'"{name}",{dev},{ts},{val:.12g}\n')
        return len(self.samples)


def main(argv=None) -> int:
    """``python -m rocm_systems_b200.tools.sysmon [-p PID ...] [--period-ms 100] [--duration S] [--fields F ...] -o out.csv [-- command]``:
    sample for ``--duration`` seconds, or for as long as the command after ``--`` runs (its process is watched too), and write
    the samples as a counter CSV that ``tools/tracedb.py import`` takes."""
    import argparse
    import subprocess
    import sys
    import time

    ap = argparse.ArgumentParser(prog="sysmon", description="Sample GPU, host and per-process counters into a CSV.")
    ap.add_argument("-p", "--pid", type=int, action="append", default=[], help="process to watch (repeatable)")
    ap.add_argument("--period-ms", type=int, default=100)
    ap.add_argument("--duration", type=float, default=0.0, help="seconds to sample when no command is given")
    ap.add_argument("--fields", nargs="+", default=list(GPU_FIELDS), help="GPU readings (names of tools/smi.py)")
    ap.add_argument("--no-gpu", action="store_true")
    ap.add_argument("-o", "--output", default="sysmon.csv")
    ap.add_argument("command", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    cmd = a.command[1:] if a.command and a.command[0] == "--" else a.command
    if not cmd and a.duration <= 0:
        ap.error("give --duration or a command after --")
    rc = 0
    child = subprocess.Popen(cmd) if cmd else None
    pids = list(a.pid) + ([child.pid] if child else [])
    with SystemSampler(period_ms=a.period_ms, pids=pids, gpu=not a.no_gpu, gpu_fields=a.fields) as s:
        if child:
            rc = child.wait()
        else:
            time.sleep(a.duration)
    n = s.write_csv(a.output)
    print(f"sysmon: {n} samples of {len({x[0] for x in s.samples})} counters in {a.output}", file=sys.stderr)
    return rc


if __name__ == "__main__":
    import sys

    sys.exit(main())
