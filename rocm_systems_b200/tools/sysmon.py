"""Background system sampler: GPU readings (through NVML), host CPU and memory, and the resident
set of chosen processes, on the same clock as the tracers, written as counter tracks.

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


class SystemSampler:
    """Background thread that samples GPU readings (NVML) and host counters at a fixed period; a context manager."""

    def __init__(self, period_ms: int = 100, pids: Sequence[int] = (), gpu: bool = True, gpu_fields: Sequence[str] = GPU_FIELDS):
        self.period = period_ms / 1e3
        self.pids = list(pids)
        self.samples: List[Tuple[str, int, int, float]] = []  # (counter, device or pid, monotonic ns, value)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.gpu_fields = list(gpu_fields)
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
        for pid in self.pids:
            r = _rss(pid)
            if r is not None:
                self.samples.append(("process_rss_bytes", pid, now, float(r)))
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
                f.write(f'"{name}",{dev},{ts},{val:.6g}\n')
        return len(self.samples)
