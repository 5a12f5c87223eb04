"""System and device dump: host, driver, every GPU's compute properties, and the peer matrix.

The counterpart of the reference's ``rocminfo`` and ``rocm_agent_enumerator``
(rocminfo/rocminfo.cc: system attributes, then one block per agent with its ISA, memory pools and
cache sizes; rocminfo/rocm_agent_enumerator: one target name per line).

    python -m rocm_systems_b200.tools.info            # full dump
    python -m rocm_systems_b200.tools.info --targets  # one "sm_XY[a]" per device, for build scripts
    python -m rocm_systems_b200.tools.info --json
"""
from __future__ import annotations

import argparse
import json
import os
import platform
import sys
from typing import Optional, Sequence


def host_info() -> dict:
    mem_kb = 0
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemTotal:"):
                    mem_kb = int(line.split()[1])
                    break
    except OSError:
        pass
    cpu = platform.processor() or ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    cpu = line.split(":", 1)[1].strip()
                    break
    except OSError:
        pass
    return {"hostname": platform.node(), "kernel": platform.release(), "cpu": cpu, "cpu_count": os.cpu_count(), "memory_bytes": mem_kb * 1024}


def arch_target(major: int, minor: int) -> str:
    """The nvcc target name; architecture-specific ('a') targets exist from Hopper on."""
    return f"sm_{major}{minor}" + ("a" if major >= 9 else "")


def device_info() -> list:
    import torch

    out = []
    if not torch.cuda.is_available():
        return out
    nvml = None
    try:
        from .smi import Smi

        nvml = Smi()
    except Exception:  # NVML missing: the CUDA properties alone are still useful
        nvml = None
    n = torch.cuda.device_count()
    for d in range(n):
        p = torch.cuda.get_device_properties(d)
        free_b, total_b = torch.cuda.mem_get_info(d)
        rec = {"index": d, "name": p.name, "target": arch_target(p.major, p.minor), "compute_capability": f"{p.major}.{p.minor}",
               "multiprocessors": p.multi_processor_count, "warp_size": getattr(p, "warp_size", 32),
               "memory_total_bytes": total_b, "memory_free_bytes": free_b, "l2_cache_bytes": getattr(p, "L2_cache_size", 0),
               "shared_memory_per_block_optin": getattr(p, "shared_memory_per_block_optin", 0),
               "shared_memory_per_multiprocessor": getattr(p, "shared_memory_per_multiprocessor", 0),
               "registers_per_multiprocessor": getattr(p, "regs_per_multiprocessor", 0),
               "max_threads_per_multiprocessor": getattr(p, "max_threads_per_multi_processor", 0),
               "uuid": str(getattr(p, "uuid", "")), "pci_bus_id": getattr(p, "pci_bus_id", -1),
               "peers": [bool(d == e or torch.cuda.can_device_access_peer(d, e)) for e in range(n)]}
        if nvml is not None:
            try:
                i = nvml.info(d)
                rec.update({"sm_clock_mhz": i["smClockMhz"], "sm_clock_max_mhz": i["smClockMaxMhz"], "mem_clock_max_mhz": i["memClockMaxMhz"],
                            "power_limit_w": i["powerLimitMilliwatt"] / 1e3, "nvlinks": i["nvlinkCount"], "nvlinks_active": i["nvlinkActive"],
                            "multicast_capable": bool(i["multicastCapable"]), "bus_id": i["busId"]})
            except RuntimeError:
                pass
        out.append(rec)
    return out


def library_info() -> dict:
    import torch

    info = {"torch": torch.__version__, "torch_cuda": torch.version.cuda}
    try:
        from ..utils import markers

        info["b200coll"] = markers.build_info()
    except Exception as e:  # library not built yet
        info["b200coll"] = f"not built ({e})"
    try:
        info["driver"] = None
        if torch.cuda.is_available():
            from .smi import Smi

            info["driver"] = Smi().driver_version() if hasattr(Smi, "driver_version") else None
    except Exception:
        pass
    return info


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="info", description=__doc__.split("\n\n")[0])
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--targets", action="store_true", help="print one nvcc target per device and nothing else")
    a = ap.parse_args(argv)
    devs = device_info()
    if a.targets:
        for d in devs:
            print(d["target"])
        return 0
    doc = {"host": host_info(), "libraries": library_info(), "devices": devs}
    if a.json:
        print(json.dumps(doc, indent=1))
        return 0
    h = doc["host"]
    print("=" * 21 + "\nSystem\n" + "=" * 21)
    print(f"Host:                  {h['hostname']}  (Linux {h['kernel']})")
    print(f"CPU:                   {h['cpu']}  x{h['cpu_count']}")
    print(f"Host memory:           {h['memory_bytes'] / 2**30:.1f} GiB")
    for k, v in doc["libraries"].items():
        print(f"{k + ':':<22} {v}")
    print("=" * 21 + "\nDevices\n" + "=" * 21)
    if not devs:
        print("no CUDA device is visible to this process")
    for d in devs:
        print(f"*******\nDevice {d['index']}\n*******")
        print(f"  Name:                    {d['name']}")
        print(f"  Target:                  {d['target']}  (compute capability {d['compute_capability']})")
        print(f"  Multiprocessors:         {d['multiprocessors']}  (warp {d['warp_size']}, {d['max_threads_per_multiprocessor']} threads, "
              f"{d['registers_per_multiprocessor']} registers each)")
        print(f"  Memory:                  {d['memory_total_bytes'] / 2**30:.1f} GiB total, {d['memory_free_bytes'] / 2**30:.1f} GiB free")
        print(f"  L2 cache:                {d['l2_cache_bytes'] / 2**20:.0f} MiB")
        print(f"  Shared memory:           {d['shared_memory_per_block_optin'] / 1024:.0f} KiB per block (opt-in), "
              f"{d['shared_memory_per_multiprocessor'] / 1024:.0f} KiB per multiprocessor")
        if "nvlinks" in d:
            print(f"  Clocks:                  SM {d['sm_clock_mhz']} / {d['sm_clock_max_mhz']} MHz, memory max {d['mem_clock_max_mhz']} MHz")
            print(f"  Power limit:             {d['power_limit_w']:.0f} W")
            print(f"  NVLink:                  {d['nvlinks_active']} of {d['nvlinks']} links active; multicast {'yes' if d['multicast_capable'] else 'no'}")
            print(f"  Bus id:                  {d['bus_id']}")
        print(f"  Peer access:             {' '.join('X' if p else '.' for p in d['peers'])}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
