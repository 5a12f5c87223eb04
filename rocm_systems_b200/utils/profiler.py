"""In-process activity tracing: kernels, memory operations and CUDA API calls of this process.

Python face of ``libb200prof.so`` (csrc/include/b200coll/prof.h), the package's counterpart of the
reference's profiling SDK buffer-tracing services
(rocprofiler-sdk/source/include/rocprofiler-sdk/buffer_tracing.h).

    from rocm_systems_b200.utils.profiler import Profiler
    with Profiler(kernels=True, memops=True) as p:
        step()
    for k in p.kernels(): print(k["name"], k["end_ns"] - k["start_ns"])
"""
from __future__ import annotations

import ctypes
from collections import defaultdict
from pathlib import Path
from typing import Dict, List

KERNEL, MEMOP, RUNTIME_API, DRIVER_API, SYNC = 1, 2, 4, 8, 16


class _Kernel(ctypes.Structure):
    _fields_ = [("start_ns", ctypes.c_uint64), ("end_ns", ctypes.c_uint64), ("device", ctypes.c_uint32), ("context", ctypes.c_uint32),
                ("stream", ctypes.c_uint32), ("correlation_id", ctypes.c_uint32), ("grid", ctypes.c_int32 * 3), ("block", ctypes.c_int32 * 3),
                ("cluster", ctypes.c_uint32 * 3), ("static_smem", ctypes.c_int32), ("dynamic_smem", ctypes.c_int32),
                ("registers", ctypes.c_uint32), ("local_per_thread", ctypes.c_uint32), ("graph_node_id", ctypes.c_uint64),
                ("name", ctypes.c_char * 192)]


class _Memop(ctypes.Structure):
    _fields_ = [("start_ns", ctypes.c_uint64), ("end_ns", ctypes.c_uint64), ("bytes", ctypes.c_uint64), ("device", ctypes.c_uint32),
                ("context", ctypes.c_uint32), ("stream", ctypes.c_uint32), ("correlation_id", ctypes.c_uint32), ("op", ctypes.c_uint8),
                ("copy_kind", ctypes.c_uint8), ("src_kind", ctypes.c_uint8), ("dst_kind", ctypes.c_uint8), ("src_device", ctypes.c_uint32),
                ("dst_device", ctypes.c_uint32)]


class _Api(ctypes.Structure):
    _fields_ = [("start_ns", ctypes.c_uint64), ("end_ns", ctypes.c_uint64), ("cbid", ctypes.c_uint32), ("pid", ctypes.c_uint32),
                ("tid", ctypes.c_uint32), ("correlation_id", ctypes.c_uint32), ("return_value", ctypes.c_uint32), ("domain", ctypes.c_uint32),
                ("name", ctypes.c_char * 64)]


_lib = None


def library_path() -> Path:
    return Path(__file__).resolve().parents[1] / "lib" / "libb200prof.so"


def load():
    global _lib
    if _lib is None:
        path = library_path()
        if not path.exists():
            raise RuntimeError(f"{path} is missing: run `python -m rocm_systems_b200.utils.build`")
        lib = ctypes.CDLL(str(path))
        lib.b200profStart.argtypes = [ctypes.c_uint]
        for fn in ("b200profKernels", "b200profMemops", "b200profApis"):
            getattr(lib, fn).argtypes = [ctypes.c_void_p, ctypes.c_uint64]
            getattr(lib, fn).restype = ctypes.c_uint64
        lib.b200profDropped.restype = ctypes.c_uint64
        lib.b200profWriteCsv.argtypes = [ctypes.c_char_p]
        lib.b200profLastError.restype = ctypes.c_char_p
        _lib = lib
    return _lib


def _rows(fn, typ) -> list:
    n = int(fn(None, 0))
    if n == 0:
        return []
    buf = (typ * n)()
    n = min(n, int(fn(buf, n)))
    return list(buf[:n])


class Profiler:
    """In-process control of the CUPTI activity tracer: ``with Profiler(kinds, output): ...`` collects and writes the records."""

    def __init__(self, kernels: bool = True, memops: bool = False, runtime_api: bool = False, driver_api: bool = False, sync: bool = False):
        self.kinds = (KERNEL if kernels else 0) | (MEMOP if memops else 0) | (RUNTIME_API if runtime_api else 0) | \
                     (DRIVER_API if driver_api else 0) | (SYNC if sync else 0)
        self.lib = load()

    def start(self) -> "Profiler":
        if self.lib.b200profStart(self.kinds) != 0:
            raise RuntimeError("b200profStart: " + self.lib.b200profLastError().decode())
        return self

    def stop(self) -> None:
        import torch

        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if self.lib.b200profStop() != 0:
            raise RuntimeError("b200profStop: " + self.lib.b200profLastError().decode())

    __enter__ = start

    def __exit__(self, *exc) -> None:
        self.stop()

    def kernels(self) -> List[dict]:
        return [{"name": k.name.decode(errors="replace"), "start_ns": k.start_ns, "end_ns": k.end_ns, "device": k.device, "stream": k.stream,
                 "correlation_id": k.correlation_id, "grid": tuple(k.grid), "block": tuple(k.block), "cluster": tuple(k.cluster),
                 "static_smem": k.static_smem, "dynamic_smem": k.dynamic_smem, "registers": k.registers,
                 "local_per_thread": k.local_per_thread, "graph_node_id": k.graph_node_id} for k in _rows(self.lib.b200profKernels, _Kernel)]

    def memops(self) -> List[dict]:
        ops = ("memcpy", "memcpy_p2p", "memset")
        return [{"op": ops[m.op] if m.op < 3 else "?", "bytes": m.bytes, "start_ns": m.start_ns, "end_ns": m.end_ns, "device": m.device,
                 "stream": m.stream, "copy_kind": m.copy_kind, "src_device": m.src_device, "dst_device": m.dst_device,
                 "correlation_id": m.correlation_id} for m in _rows(self.lib.b200profMemops, _Memop)]

    def apis(self) -> List[dict]:
        return [{"name": a.name.decode(errors="replace"), "start_ns": a.start_ns, "end_ns": a.end_ns, "tid": a.tid, "domain": a.domain,
                 "correlation_id": a.correlation_id, "return_value": a.return_value} for a in _rows(self.lib.b200profApis, _Api)]

    def dropped(self) -> int:
        return int(self.lib.b200profDropped())

    def clear(self) -> None:
        self.lib.b200profClear()

    def write_csv(self, prefix: str) -> int:
        return int(self.lib.b200profWriteCsv(prefix.encode()))

    def kernel_summary(self) -> Dict[str, dict]:
        """name -> {calls, total_ns, mean_ns, min_ns, max_ns}, the per-kernel statistics table."""
        acc: Dict[str, list] = defaultdict(list)
        for k in self.kernels():
            acc[k["name"]].append(k["end_ns"] - k["start_ns"])
        return {n: {"calls": len(v), "total_ns": sum(v), "mean_ns": sum(v) / len(v), "min_ns": min(v), "max_ns": max(v)} for n, v in acc.items()}


class HostSampler:
    """In-process call-stack sampling of this process's host threads (``libb200sample.so``, csrc/prof/sampler.cc): the
    part of the reference's system profiler that samples call stacks on a CPU-time or a wall-clock timer
    (rocprofiler-systems source/lib/rocprof-sys/library/sampling.cpp).

        with HostSampler(freq_hz=200, clock="wall") as s:
            step()
        s.write("out/step")            # out/step.samples.csv, out/step.folded
        for fn, share in s.top(5): ...

    One sampler per process at a time. Native frames only: Python code shows up as the interpreter's own functions.
    """

    _lib = None

    def __init__(self, freq_hz: float = 100.0, clock: str = "cpu"):
        assert clock in ("cpu", "wall")
        self.freq_hz, self.clock = float(freq_hz), clock
        if HostSampler._lib is None:
            path = Path(__file__).resolve().parents[1] / "lib" / "libb200sample.so"
            if not path.exists():
                raise RuntimeError(f"{path} is missing: run `python -m rocm_systems_b200.utils.build`")
            lib = ctypes.CDLL(str(path))
            lib.b200sampleStart.argtypes = [ctypes.c_double, ctypes.c_int]
            lib.b200sampleCount.restype = ctypes.c_uint64
            lib.b200sampleDropped.restype = ctypes.c_uint64
            lib.b200sampleWrite.argtypes = [ctypes.c_char_p]
            HostSampler._lib = lib

    def start(self) -> "HostSampler":
        HostSampler._lib.b200sampleClear()
        rc = HostSampler._lib.b200sampleStart(self.freq_hz, 0 if self.clock == "cpu" else 1)
        if rc != 0:
            raise RuntimeError(f"host sampler did not start (code {rc}: -1 already running, -2 bad argument, -4/-5 signal or timer set-up)")
        return self

    def stop(self) -> None:
        HostSampler._lib.b200sampleStop()

    __enter__ = start

    def __exit__(self, *exc) -> None:
        self.stop()

    def count(self) -> int:
        return int(HostSampler._lib.b200sampleCount())

    def dropped(self) -> int:
        return int(HostSampler._lib.b200sampleDropped())

    def write(self, prefix: str) -> int:
        rc = HostSampler._lib.b200sampleWrite(str(prefix).encode())
        if rc < 0:
            raise RuntimeError(f"host sampler could not write {prefix}.* (code {rc})")
        return rc

    def top(self, n: int = 10) -> List[tuple]:
        """(innermost function, share of samples) for the ``n`` most sampled functions."""
        import tempfile

        with tempfile.TemporaryDirectory() as d:
            self.write(f"{d}/s")
            leaf: Dict[str, int] = defaultdict(int)
            for line in Path(f"{d}/s.folded").read_text().splitlines():
                stack, _, cnt = line.rpartition(" ")
                leaf[stack.rsplit(";", 1)[-1]] += int(cnt)
        total = sum(leaf.values()) or 1
        return [(fn, c / total) for fn, c in sorted(leaf.items(), key=lambda kv: -kv[1])[:n]]
