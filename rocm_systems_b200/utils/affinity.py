"""CPU placement of the process that drives a GPU: run on the CPUs (and allocate from the NUMA node) the GPU is attached
to, so that launches, host staging buffers and the bootstrap threads do not cross the socket interconnect.

    from rocm_systems_b200.utils import affinity
    affinity.pin_to_gpu(local_rank)            # os.sched_setaffinity to the GPU's CPUs; returns what was set

The CPUs come from NVML (``b200smi_cpu_affinity``), else from the PCI device's ``local_cpulist`` in sysfs. Only CPUs the
process is already allowed on are kept (a container's cpuset wins); nothing happens when that leaves none. The reference
exposes the same facts through its management library (rocm_smi_lib ``rsmi_topo_get_numa_node_number``,
``rsmi_topo_numa_affinity_get``; ``rocm-smi --showtoponuma``) and its runtime's topology
(rocr-runtime core/runtime/amd_topology.cpp: the CPU agent nearest to a GPU agent); collective libraries use them to pin
their helper threads.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence


def parse_cpu_list(text: str) -> List[int]:
    """``"0-3,8,10-11"`` -> ``[0, 1, 2, 3, 8, 10, 11]``."""
    out: List[int] = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        lo, dash, hi = part.partition("-")
        out += list(range(int(lo), int(hi) + 1)) if dash else [int(lo)]
    return out


def format_cpu_list(cpus: Sequence[int]) -> str:
    """The inverse: ranges joined by commas."""
    out, run = [], []
    for c in sorted(set(cpus)):
        if run and c == run[-1] + 1:
            run.append(c)
        else:
            if run:
                out.append(run)
            run = [c]
    if run:
        out.append(run)
    return ",".join(str(r[0]) if len(r) == 1 else f"{r[0]}-{r[-1]}" for r in out)


def gpu_cpus(device: int, sysfs_root: str = "/sys") -> Dict[str, object]:
    """``{"cpus": [...], "numa_node": n or None, "source": "nvml" | "sysfs" | "none"}`` for a CUDA device index."""
    bus_id = None
    try:
        from ..tools.smi import Smi

        s = Smi()
        try:
            bus_id = s.info(device)["busId"]
            a = s.cpu_affinity(device)
            if a["cpus"]:
                return {"cpus": a["cpus"], "numa_node": a["numa_node"], "source": "nvml"}
        finally:
            s.close()
    except (RuntimeError, OSError, AttributeError):
        pass
    if bus_id:
        # NVML prints an 8-digit PCI domain, sysfs a 4-digit one
        short = bus_id.lower()
        if len(short.split(":")[0]) == 8:
            short = short[4:]
        base = os.path.join(sysfs_root, "bus", "pci", "devices", short)
        try:
            cpus = parse_cpu_list(open(os.path.join(base, "local_cpulist")).read())
            node = int(open(os.path.join(base, "numa_node")).read().strip())
            if cpus:
                return {"cpus": cpus, "numa_node": node if node >= 0 else None, "source": "sysfs"}
        except (OSError, ValueError):
            pass
    return {"cpus": [], "numa_node": None, "source": "none"}


def pin_to_gpu(device: int, sysfs_root: str = "/sys", pid: int = 0) -> Optional[List[int]]:
    """Restricts the process (all its current threads' default, and threads started later) to the CPUs of ``device`` that it
    is already allowed on. Returns the CPUs set, or None when nothing was changed."""
    local = gpu_cpus(device, sysfs_root)["cpus"]
    if not local:
        return None
    allowed = os.sched_getaffinity(pid)
    target = sorted(set(local) & allowed)
    if not target or set(target) == allowed:
        return None
    os.sched_setaffinity(pid, target)
    return target


def wanted() -> bool:
    """True when the environment asks for pinning (``B200COLL_CPU_AFFINITY=1``)."""
    return os.environ.get("B200COLL_CPU_AFFINITY", "0").strip().lower() in ("1", "true", "yes", "on")
