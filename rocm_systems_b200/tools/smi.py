"""``b200-smi``: device readings and topology tables, the CLI counterpart of rocm-smi
(rocm-smi-lib/python_smi_tools/rocm_smi.py: showWeightTopology :3279, showHopsTopology :3326,
showTypeTopology :3372, showNodesBw :3460) on top of the native ``b200smi_*`` API.

    python -m rocm_systems_b200.tools.smi --showall
    python -m rocm_systems_b200.tools.smi --showtopo [--json]
    python -m rocm_systems_b200.tools.smi metric -g 0 1 --csv        # subcommands: version list static metric topology process monitor event

Setters (``--setpowerlimit``, ``--setclocks``, ``--resetclocks``) do nothing unless ``--allow-set`` is given AND B200SMI_ALLOW_SET=1 is
in the environment; GPUs on shared hosts must be left as they were found.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import sys

from .. import _lib

FIELDS = {"sm_clock": 1, "mem_clock": 2, "power": 3, "temp": 4, "mem_used": 5, "gpu_util": 6, "mem_util": 7, "ecc_corrected": 8,
          "ecc_uncorrected": 9, "throttle_reasons": 10, "nvlink_active": 11,
          # activity over the interval since the previous reading (percent of peak; MiB/s)
          "sm_active": 12, "sm_occupancy": 13, "tensor_active": 14, "dram_active": 15, "fp64_active": 16, "fp32_active": 17, "fp16_active": 18,
          "pcie_tx_mibs": 19, "pcie_rx_mibs": 20, "nvlink_tx_mibs": 21, "nvlink_rx_mibs": 22}
ACTIVITY_FIELDS = [f for f, i in FIELDS.items() if i >= 12]
REASON_BITS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
               0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}
LINK_TYPES = {0: "SELF", 1: "NVLINK", 2: "PCIE", 3: "UNKNOWN"}


class DeviceInfo(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 96), ("uuid", ctypes.c_char * 96), ("busId", ctypes.c_char * 32),
                ("smClockMhz", ctypes.c_uint32), ("smClockMaxMhz", ctypes.c_uint32), ("memClockMhz", ctypes.c_uint32), ("memClockMaxMhz", ctypes.c_uint32),
                ("powerMilliwatt", ctypes.c_uint32), ("powerLimitMilliwatt", ctypes.c_uint32), ("temperatureC", ctypes.c_uint32),
                ("memTotalBytes", ctypes.c_uint64), ("memUsedBytes", ctypes.c_uint64), ("eccCorrected", ctypes.c_uint64), ("eccUncorrected", ctypes.c_uint64),
                ("throttleReasons", ctypes.c_uint64), ("gpuUtilPct", ctypes.c_uint32), ("memUtilPct", ctypes.c_uint32),
                ("nvlinkCount", ctypes.c_uint32), ("nvlinkActive", ctypes.c_uint32), ("multicastCapable", ctypes.c_uint32)]


class Link(ctypes.Structure):
    _fields_ = [("type", ctypes.c_int), ("hops", ctypes.c_uint32), ("weight", ctypes.c_uint32), ("nvlinks", ctypes.c_uint32),
                ("minBandwidthMBps", ctypes.c_uint64), ("maxBandwidthMBps", ctypes.c_uint64), ("p2pAccessible", ctypes.c_int),
                ("atomics32", ctypes.c_int), ("atomics64", ctypes.c_int), ("coherent", ctypes.c_int), ("perfRank", ctypes.c_int)]


class Sample(ctypes.Structure):
    _fields_ = [("timestampNs", ctypes.c_uint64), ("value", ctypes.c_double)]


class Stats(ctypes.Structure):
    _fields_ = [("min", ctypes.c_double), ("max", ctypes.c_double), ("avg", ctypes.c_double), ("last", ctypes.c_double), ("samples", ctypes.c_uint64)]


class Process(ctypes.Structure):
    _fields_ = [("pid", ctypes.c_uint32), ("usedMemoryBytes", ctypes.c_uint64), ("name", ctypes.c_char * 64)]


class NvlinkErrors(ctypes.Structure):
    _fields_ = [("replay", ctypes.c_uint64), ("recovery", ctypes.c_uint64), ("crcFlit", ctypes.c_uint64), ("crcData", ctypes.c_uint64),
                ("linksRead", ctypes.c_uint32)]


class Modes(ctypes.Structure):
    _fields_ = [("computeMode", ctypes.c_int), ("persistence", ctypes.c_int), ("mig", ctypes.c_int), ("ecc", ctypes.c_int)]


POLICY_CB = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_int, ctypes.c_double, ctypes.c_double, ctypes.c_void_p)


class Event(ctypes.Structure):
    _fields_ = [("device", ctypes.c_int), ("type", ctypes.c_uint64), ("data", ctypes.c_uint64), ("timestampNs", ctypes.c_uint64)]


EVENT_NAMES = {0x1: "ecc_single_bit", 0x2: "ecc_double_bit", 0x4: "pstate", 0x8: "xid", 0x10: "clock", 0x80: "power_source"}
ERR_TIMEOUT = 6


class Identity(ctypes.Structure):
    _fields_ = [("serial", ctypes.c_char * 32), ("partNumber", ctypes.c_char * 64), ("vbios", ctypes.c_char * 32), ("inforomImage", ctypes.c_char * 32),
                ("performanceState", ctypes.c_int), ("powerLimitMinMilliwatt", ctypes.c_int64), ("powerLimitMaxMilliwatt", ctypes.c_int64),
                ("energyMillijoule", ctypes.c_int64), ("remappedCorrectable", ctypes.c_int), ("remappedUncorrectable", ctypes.c_int),
                ("remapPending", ctypes.c_int), ("remapFailed", ctypes.c_int)]


class Activity(ctypes.Structure):
    _fields_ = [(n, ctypes.c_double) for n in ("intervalMs", "smActivePct", "smOccupancyPct", "tensorActivePct", "dramActivePct", "fp64ActivePct",
                                                "fp32ActivePct", "fp16ActivePct", "pcieTxMiBs", "pcieRxMiBs", "nvlinkTxMiBs", "nvlinkRxMiBs")]


class Smi:
    """Thin object wrapper over the C API; raises RuntimeError with the library's message."""

    def __init__(self):
        self.lib = _lib.load()
        L = self.lib
        L.b200smi_status_string.restype = ctypes.c_char_p
        L.b200smi_device_info.argtypes = [ctypes.c_int, ctypes.POINTER(DeviceInfo)]
        L.b200smi_link.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(Link)]
        L.b200smi_read_field.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
        L.b200smi_watch_latest.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(Sample)]
        L.b200smi_watch_history.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(Sample), ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        L.b200smi_job_stats.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(Stats)]
        L.b200smi_policy_set.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_double, ctypes.c_int, POLICY_CB, ctypes.c_void_p]
        L.b200smi_health.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_char_p, ctypes.c_int]
        L.b200smi_set_power_limit.argtypes = [ctypes.c_int, ctypes.c_uint32, ctypes.c_int]
        L.b200smi_driver_version.argtypes = [ctypes.c_char_p, ctypes.c_int]
        L.b200smi_processes.argtypes = [ctypes.c_int, ctypes.POINTER(Process), ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        L.b200smi_nvlink_errors.argtypes = [ctypes.c_int, ctypes.POINTER(NvlinkErrors)]
        L.b200smi_modes.argtypes = [ctypes.c_int, ctypes.POINTER(Modes)]
        L.b200smi_pcie.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint32)]
        L.b200smi_events_open.argtypes = [ctypes.c_uint64]
        L.b200smi_events_wait.argtypes = [ctypes.c_int, ctypes.POINTER(Event)]
        self._cbs = []
        self._ck(L.b200smi_init())

    def _ck(self, st: int) -> None:
        if st != 0:
            raise RuntimeError(self.lib.b200smi_status_string(st).decode())

    def close(self) -> None:
        self.lib.b200smi_shutdown()

    def count(self) -> int:
        n = ctypes.c_int()
        self._ck(self.lib.b200smi_device_count(ctypes.byref(n)))
        return n.value

    def info(self, dev: int) -> dict:
        i = DeviceInfo()
        self._ck(self.lib.b200smi_device_info(dev, ctypes.byref(i)))
        d = {f[0]: getattr(i, f[0]) for f in DeviceInfo._fields_}
        for k in ("name", "uuid", "busId"):
            d[k] = d[k].decode()
        d["throttleReasonNames"] = [n for b, n in REASON_BITS.items() if d["throttleReasons"] & b]
        return d

    def link(self, a: int, b: int) -> dict:
        l = Link()
        self._ck(self.lib.b200smi_link(a, b, ctypes.byref(l)))
        d = {f[0]: getattr(l, f[0]) for f in Link._fields_}
        d["typeName"] = LINK_TYPES.get(d["type"], "UNKNOWN")
        return d

    def read(self, dev: int, field: str) -> float:
        v = ctypes.c_double()
        self._ck(self.lib.b200smi_read_field(dev, FIELDS[field], ctypes.byref(v)))
        return v.value

    def watch_start(self, devs, fields, period_ms=1000, keep=600) -> None:
        da = (ctypes.c_int * len(devs))(*devs)
        fa = (ctypes.c_int * len(fields))(*[FIELDS[f] for f in fields])
        self._ck(self.lib.b200smi_watch_start(da, len(devs), fa, len(fields), period_ms, keep))

    def watch_stop(self) -> None:
        self.lib.b200smi_watch_stop()

    def history(self, dev: int, field: str, max_n: int = 4096):
        n = ctypes.c_int()
        arr = (Sample * max_n)()
        self._ck(self.lib.b200smi_watch_history(dev, FIELDS[field], arr, max_n, ctypes.byref(n)))
        return [(arr[i].timestampNs, arr[i].value) for i in range(min(n.value, max_n))]

    def job_start(self, job: str) -> None:
        self._ck(self.lib.b200smi_job_start(job.encode()))

    def job_stop(self, job: str) -> None:
        self._ck(self.lib.b200smi_job_stop(job.encode()))

    def job_stats(self, job: str, dev: int, field: str) -> dict:
        s = Stats()
        self._ck(self.lib.b200smi_job_stats(job.encode(), dev, FIELDS[field], ctypes.byref(s)))
        return {f[0]: getattr(s, f[0]) for f in Stats._fields_}

    def policy(self, dev: int, field: str, threshold: float, above: bool, fn) -> None:
        cb = POLICY_CB(lambda d, f, v, t, u: fn(d, f, v, t))
        self._cbs.append(cb)
        self._ck(self.lib.b200smi_policy_set(dev, FIELDS[field], threshold, 1 if above else -1, cb, None))

    def health(self, dev: int):
        lv = ctypes.c_int()
        buf = ctypes.create_string_buffer(256)
        self._ck(self.lib.b200smi_health(dev, ctypes.byref(lv), buf, 256))
        return lv.value, buf.value.decode()

    def driver_version(self) -> str:
        buf = ctypes.create_string_buffer(96)
        self._ck(self.lib.b200smi_driver_version(buf, 96))
        return buf.value.decode()

    def processes(self, dev: int) -> list:
        """Compute processes on the device: pid, device memory in use, command name."""
        n = ctypes.c_int()
        arr = (Process * 256)()
        self._ck(self.lib.b200smi_processes(dev, arr, 256, ctypes.byref(n)))
        return [{"pid": arr[i].pid, "used_memory_bytes": arr[i].usedMemoryBytes, "name": arr[i].name.decode(errors="replace")}
                for i in range(min(n.value, 256))]

    def nvlink_errors(self, dev: int) -> dict:
        e = NvlinkErrors()
        self._ck(self.lib.b200smi_nvlink_errors(dev, ctypes.byref(e)))
        return {f[0]: getattr(e, f[0]) for f in NvlinkErrors._fields_}

    def activity(self, dev: int) -> dict:
        """Activity since the previous call for this device (the first call measures 100 ms itself): SM busy, occupancy,
        tensor / DRAM / FP pipes in percent of peak, PCIe and NVLink traffic in MiB/s; ``None`` where the device reports
        nothing. Raises when the driver has no performance-monitoring samples."""
        a = Activity()
        self.lib.b200smi_activity.argtypes = [ctypes.c_int, ctypes.POINTER(Activity)]
        self._ck(self.lib.b200smi_activity(dev, ctypes.byref(a)))
        names = {"intervalMs": "interval_ms", "smActivePct": "sm_active_pct", "smOccupancyPct": "sm_occupancy_pct", "tensorActivePct": "tensor_active_pct",
                 "dramActivePct": "dram_active_pct", "fp64ActivePct": "fp64_active_pct", "fp32ActivePct": "fp32_active_pct", "fp16ActivePct": "fp16_active_pct",
                 "pcieTxMiBs": "pcie_tx_mibs", "pcieRxMiBs": "pcie_rx_mibs", "nvlinkTxMiBs": "nvlink_tx_mibs", "nvlinkRxMiBs": "nvlink_rx_mibs"}
        return {names[f[0]]: (None if getattr(a, f[0]) < 0 else round(getattr(a, f[0]), 3)) for f in Activity._fields_}

    def pcie(self, dev: int) -> dict:
        g, w = ctypes.c_uint32(), ctypes.c_uint32()
        self._ck(self.lib.b200smi_pcie(dev, ctypes.byref(g), ctypes.byref(w)))
        return {"generation": g.value, "width": w.value}

    def modes(self, dev: int) -> dict:
        """Compute / persistence / MIG / ECC modes as the driver reports them (read only; -1 = not reported)."""
        m = Modes()
        self._ck(self.lib.b200smi_modes(dev, ctypes.byref(m)))
        names = {0: "default", 1: "exclusive_thread", 2: "prohibited", 3: "exclusive_process"}
        return {"compute_mode": names.get(m.computeMode, str(m.computeMode)), "persistence": m.persistence, "mig": m.mig, "ecc": m.ecc}

    def events(self, timeout_ms: int = 1000, mask: int = 0, max_events: int = 0, stop=None):
        """Yields asynchronous device events (XID errors, ECC errors, power-state and clock changes) as dicts until
        ``timeout_ms`` passes without one, or ``max_events`` have been seen. With ``stop`` (a ``threading.Event``) quiet
        periods do not end the stream: it runs, on one event set, until ``stop`` is set. Read only."""
        self._ck(self.lib.b200smi_events_open(mask))
        try:
            seen = 0
            while not max_events or seen < max_events:
                ev = Event()
                st = self.lib.b200smi_events_wait(timeout_ms, ctypes.byref(ev))
                if st == ERR_TIMEOUT:
                    if stop is not None and not stop.is_set():
                        continue
                    return
                self._ck(st)
                seen += 1
                yield {"device": ev.device, "type": EVENT_NAMES.get(ev.type, hex(ev.type)), "data": ev.data, "timestamp_ns": ev.timestampNs}
        finally:
            self.lib.b200smi_events_close()

    def set_power_limit(self, dev: int, milliwatt: int, allow: bool) -> None:
        self._ck(self.lib.b200smi_set_power_limit(dev, milliwatt, int(allow)))

    def set_locked_clocks(self, dev: int, min_mhz: int, max_mhz: int, allow: bool) -> None:
        """Locks the SM clock into a range (outlasts the process: reset it afterwards). Refused unless allowed twice over."""
        self.lib.b200smi_set_locked_clocks.argtypes = [ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int]
        self._ck(self.lib.b200smi_set_locked_clocks(dev, min_mhz, max_mhz, int(allow)))

    def reset_locked_clocks(self, dev: int, allow: bool) -> None:
        self.lib.b200smi_reset_locked_clocks.argtypes = [ctypes.c_int, ctypes.c_int]
        self._ck(self.lib.b200smi_reset_locked_clocks(dev, int(allow)))

    def cpu_affinity(self, dev: int) -> dict:
        """``{"cpus": [...], "numa_node": n or None}``: the logical CPUs (and NUMA node) the device is attached to."""
        words = 16
        mask = (ctypes.c_uint64 * words)()
        node = ctypes.c_int(-1)
        self.lib.b200smi_cpu_affinity.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_uint64), ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        self._ck(self.lib.b200smi_cpu_affinity(dev, mask, words, ctypes.byref(node)))
        cpus = [w * 64 + b for w in range(words) for b in range(64) if mask[w] >> b & 1]
        return {"cpus": cpus, "numa_node": None if node.value < 0 else node.value}

    def identity(self, dev: int) -> dict:
        """Serial and part number, firmware versions, performance state, settable power range (W), energy since the driver
        loaded (J), remapped memory rows; ``None`` where the driver reports nothing."""
        i = Identity()
        self.lib.b200smi_identity.argtypes = [ctypes.c_int, ctypes.POINTER(Identity)]
        self._ck(self.lib.b200smi_identity(dev, ctypes.byref(i)))
        text = lambda b: b.decode(errors="replace") or None  # noqa: E731
        num = lambda v, scale=1: None if v < 0 else v / scale  # noqa: E731
        return {"serial": text(i.serial), "part_number": text(i.partNumber), "vbios": text(i.vbios), "inforom_image": text(i.inforomImage),
                "performance_state": None if i.performanceState < 0 else i.performanceState,
                "power_limit_min_w": num(i.powerLimitMinMilliwatt, 1000), "power_limit_max_w": num(i.powerLimitMaxMilliwatt, 1000),
                "energy_j": num(i.energyMillijoule, 1000),
                "remapped_rows": None if i.remappedCorrectable < 0 else {"correctable": i.remappedCorrectable, "uncorrectable": i.remappedUncorrectable,
                                                                          "pending": bool(i.remapPending), "failed": bool(i.remapFailed)}}


def _matrix(smi: Smi, key: str, n: int):
    return [[smi.link(i, j)[key] for j in range(n)] for i in range(n)]


def _print_matrix(title: str, m, n: int) -> None:
    print(f"\n=== {title} ===")
    print("       " + "".join(f"GPU{j:<9}" for j in range(n)))
    for i in range(n):
        print(f"GPU{i:<4}" + "".join(f"{str(m[i][j]):<12}" for j in range(n)))


SUBCOMMANDS = ("version", "list", "static", "firmware", "bad-pages", "metric", "nvlink", "topology", "process", "monitor", "event", "set", "reset")


def _sub_main(argv) -> int:
    """The subcommand front end (the layout of the reference's newer amd-smi command line: ``list``, ``static``, ``metric``,
    ``firmware``, ``bad-pages``, ``xgmi`` (here ``nvlink``), ``topology``, ``process``, ``monitor``, ``event``, ``set``, ``reset``,
    ``version``), over the same readings as the flag front end. Every subcommand takes ``-g GPU [GPU ...]`` and ``--json`` /
    ``--csv``. Only ``set`` and ``reset`` can change a device, and only with ``--allow-set`` and B200SMI_ALLOW_SET=1; ``reset``
    hands locked clocks back to the driver, it never resets a GPU."""
    ap = argparse.ArgumentParser(prog="b200-smi")
    sub = ap.add_subparsers(dest="cmd", required=True)
    subs = {}
    for name, help_ in (("version", "tool, library and driver versions"), ("list", "index, bus id and UUID of every GPU"),
                        ("static", "what does not change while the GPU runs: product, bus, limits, modes, link count"),
                        ("metric", "what does: clocks, power, temperature, memory, utilisation, ECC totals, NVLink error counters, throttle reasons"),
                        ("topology", "link type, hops, weight, bandwidth and peer access between every pair"),
                        ("firmware", "VBIOS and InfoROM image versions"), ("bad-pages", "rows of device memory remapped after errors"),
                        ("nvlink", "links up, error counters and, with --activity, traffic per GPU"),
                        ("set", "power limit or SM clock range (refused unless allowed twice over)"), ("reset", "hand locked SM clocks back to the driver"),
                        ("process", "compute processes per GPU"), ("monitor", "one line of readings per GPU and interval"),
                        ("event", "XID / ECC / power-state / clock events as they happen")):
        sp = sub.add_parser(name, help=help_)
        sp.add_argument("-g", "--gpu", nargs="+", type=int, default=None, help="GPU indices (default: all)")
        sp.add_argument("--json", action="store_true")
        sp.add_argument("--csv", action="store_true")
        subs[name] = sp
    subs["monitor"].add_argument("-w", "--watch", type=float, default=1.0, metavar="SECONDS", help="interval between lines")
    subs["monitor"].add_argument("-i", "--iterations", type=int, default=1, help="how many intervals (0: until interrupted)")
    subs["set"].add_argument("--power-limit", type=float, metavar="WATTS")
    subs["set"].add_argument("--clocks", type=int, nargs=2, metavar=("MIN_MHZ", "MAX_MHZ"))
    subs["reset"].add_argument("--clocks", action="store_true", help="the only thing that can be reset")
    for name in ("set", "reset"):
        subs[name].add_argument("--allow-set", action="store_true", help="required, together with B200SMI_ALLOW_SET=1")
    for name in ("metric", "monitor", "nvlink"):
        subs[name].add_argument("--activity", action="store_true", help="SM / tensor / DRAM activity and PCIe / NVLink traffic over the interval "
                                "(performance-monitoring samples of the driver; no profiler involved)")
    subs["event"].add_argument("-t", "--timeout", type=float, default=5.0, metavar="SECONDS", help="stop after this long without an event")
    a = ap.parse_args(argv)
    try:
        smi = Smi()
    except RuntimeError as e:
        print(f"b200-smi: {e}", file=sys.stderr)
        return 1
    n = smi.count()
    gpus = [g for g in (a.gpu if a.gpu is not None else range(n))]
    bad = [g for g in gpus if not 0 <= g < n]
    if bad:
        print(f"b200-smi: no GPU {bad[0]} (there are {n})", file=sys.stderr)
        smi.close()
        return 2

    def emit(rows):
        """rows: a list of flat dicts (one per GPU, pair or process)."""
        if a.json:
            print(json.dumps(rows, indent=1))
        elif a.csv:
            import csv as _csv

            keys = list(dict.fromkeys(k for r in rows for k in r))
            w = _csv.writer(sys.stdout)
            w.writerow(keys)
            for r in rows:
                w.writerow([r.get(k, "") for k in keys])
        else:
            for r in rows:
                head = f"GPU {r['gpu']}" if "gpu" in r else ""
                print((head + ": " if head else "") + ", ".join(f"{k} {v}" for k, v in r.items() if k != "gpu"))

    if a.cmd == "version":
        from .. import __version__

        emit([{"tool": "b200-smi", "package": __version__, "driver": smi.driver_version()}])
    elif a.cmd == "list":
        emit([{"gpu": g, "bus_id": smi.info(g)["busId"], "uuid": smi.info(g)["uuid"]} for g in gpus])
    elif a.cmd == "firmware":
        emit([{"gpu": g, "vbios": smi.identity(g)["vbios"], "inforom_image": smi.identity(g)["inforom_image"], "driver": smi.driver_version()} for g in gpus])
    elif a.cmd == "bad-pages":
        rows = []
        for g in gpus:
            r = smi.identity(g)["remapped_rows"]
            rows.append({"gpu": g, **(r if r is not None else {"correctable": None, "uncorrectable": None, "pending": None, "failed": None})})
        emit(rows)
    elif a.cmd == "nvlink":
        rows = []
        for g in gpus:
            d, e = smi.info(g), smi.nvlink_errors(g)
            rows.append({"gpu": g, "links": d["nvlinkCount"], "links_up": d["nvlinkActive"], "replay": e["replay"], "recovery": e["recovery"],
                         "crc_flit": e["crcFlit"], "crc_data": e["crcData"]})
            if a.activity:
                act = smi.activity(g)
                rows[-1].update({"tx_mibs": act["nvlink_tx_mibs"], "rx_mibs": act["nvlink_rx_mibs"]})
        emit(rows)
    elif a.cmd in ("set", "reset"):
        try:
            for g in gpus if a.gpu is not None else []:
                if a.cmd == "set" and a.power_limit is not None:
                    smi.set_power_limit(g, int(a.power_limit * 1000), a.allow_set)
                if a.cmd == "set" and a.clocks:
                    smi.set_locked_clocks(g, a.clocks[0], a.clocks[1], a.allow_set)
                if a.cmd == "reset" and a.clocks:
                    smi.reset_locked_clocks(g, a.allow_set)
            if a.gpu is None:
                print("b200-smi: name the GPUs with -g; nothing is set on all GPUs by default", file=sys.stderr)
                smi.close()
                return 2
            emit([{"gpu": g, "done": a.cmd} for g in gpus])
        except RuntimeError as e:
            print(f"b200-smi: {e}", file=sys.stderr)
            smi.close()
            return 2
    elif a.cmd == "static":
        rows = []
        for g in gpus:
            d, m, pc, ident = smi.info(g), smi.modes(g), smi.pcie(g), smi.identity(g)
            rows.append({"gpu": g, "name": d["name"], "bus_id": d["busId"], "uuid": d["uuid"], "serial": ident["serial"], "part_number": ident["part_number"],
                         "vbios": ident["vbios"], "power_limit_range_w": None if ident["power_limit_max_w"] is None else
                         f"{ident['power_limit_min_w']:.0f}-{ident['power_limit_max_w']:.0f}", "memory_total_gib": round(d["memTotalBytes"] / 2**30, 1),
                         "sm_clock_max_mhz": d["smClockMaxMhz"], "memory_clock_max_mhz": d["memClockMaxMhz"], "power_limit_w": d["powerLimitMilliwatt"] / 1000,
                         "pcie_generation": pc["generation"], "pcie_width": pc["width"], "nvlink_links": d["nvlinkCount"], "compute_mode": m["compute_mode"],
                         "persistence": m["persistence"], "mig": m["mig"], "ecc": m["ecc"]})
        emit(rows)
    elif a.cmd == "metric":
        rows = []
        for g in gpus:
            d, e = smi.info(g), smi.nvlink_errors(g)
            rows.append({"gpu": g, "sm_clock_mhz": d["smClockMhz"], "memory_clock_mhz": d["memClockMhz"], "power_w": round(d["powerMilliwatt"] / 1000, 1),
                         "temperature_c": d["temperatureC"], "memory_used_gib": round(d["memUsedBytes"] / 2**30, 2), "gpu_util_pct": d["gpuUtilPct"],
                         "memory_util_pct": d["memUtilPct"], "ecc_corrected": d["eccCorrected"], "ecc_uncorrected": d["eccUncorrected"],
                         "nvlink_active": d["nvlinkActive"], "nvlink_replay": e["replay"], "nvlink_recovery": e["recovery"], "nvlink_crc": e["crcFlit"] + e["crcData"],
                         "throttle": ",".join(d["throttleReasonNames"]) or "none"})
            if a.activity:
                rows[-1].update({k: v for k, v in smi.activity(g).items() if k != "interval_ms"})
        emit(rows)
    elif a.cmd == "topology":
        rows = []
        for x in gpus:
            for y in gpus:
                if x != y:
                    l = smi.link(x, y)
                    rows.append({"gpu": x, "peer": y, "type": l["typeName"], "hops": l["hops"], "weight": l["weight"], "max_bandwidth_mbps": l["maxBandwidthMBps"],
                                 "peer_access": bool(l["p2pAccessible"])})
        emit(rows)
    elif a.cmd == "process":
        emit([{"gpu": g, "pid": pr["pid"], "name": pr["name"], "memory_gib": round(pr["used_memory_bytes"] / 2**30, 2)} for g in gpus for pr in smi.processes(g)])
    elif a.cmd == "monitor":
        import time

        i = 0
        try:
            while a.iterations == 0 or i < a.iterations:
                rows = []
                for g in gpus:
                    d = smi.info(g)
                    rows.append({"gpu": g, "power_w": round(d["powerMilliwatt"] / 1000, 1), "temperature_c": d["temperatureC"], "sm_clock_mhz": d["smClockMhz"],
                                 "gpu_util_pct": d["gpuUtilPct"], "memory_util_pct": d["memUtilPct"], "memory_used_gib": round(d["memUsedBytes"] / 2**30, 2)})
                    if a.activity:   # over the interval since the previous line
                        act = smi.activity(g)
                        rows[-1].update({k: act[k] for k in ("sm_active_pct", "tensor_active_pct", "dram_active_pct", "nvlink_tx_mibs", "nvlink_rx_mibs")})
                emit(rows)
                i += 1
                if a.iterations == 0 or i < a.iterations:
                    time.sleep(max(0.0, a.watch))
        except KeyboardInterrupt:
            pass
    elif a.cmd == "event":
        rows = [ev for ev in smi.events(timeout_ms=int(a.timeout * 1000)) if ev["device"] in gpus]
        emit([{"gpu": ev["device"], "type": ev["type"], "data": ev["data"], "timestamp_ns": ev["timestamp_ns"]} for ev in rows])
    smi.close()
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] in SUBCOMMANDS:
        return _sub_main(argv)
    ap = argparse.ArgumentParser(prog="b200-smi", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--showall", action="store_true")
    ap.add_argument("--showtopo", action="store_true", help="weight, hops, type and bandwidth tables")
    ap.add_argument("--showtopoweight", action="store_true", help="only the weight table")
    ap.add_argument("--showtopohops", action="store_true", help="only the hops table")
    ap.add_argument("--showtopotype", action="store_true", help="only the link-type table")
    ap.add_argument("--showtopoaccess", action="store_true", help="only the peer-accessibility table")
    ap.add_argument("--shownodesbw", action="store_true", help="only the bandwidth table")
    ap.add_argument("--showhealth", action="store_true")
    for flag, help_ in (("--showtemp", "temperature"), ("--showpower", "power draw and limit"), ("--showclocks", "SM and memory clocks, current / max"),
                        ("--showmeminfo", "memory used / total"), ("--showuse", "GPU and memory utilisation"), ("--showuniqueid", "UUID"),
                        ("--showproductname", "product name"), ("--showecc", "ECC error totals"), ("--showthrottle", "active clock event reasons")):
        ap.add_argument(flag, action="store_true", help=help_ + " (one line per GPU)")
    ap.add_argument("--showpids", action="store_true", help="compute processes per GPU")
    ap.add_argument("--showdriverversion", action="store_true")
    ap.add_argument("--shownvlinkerrors", action="store_true", help="replay / recovery / CRC counters summed over each GPU's links")
    ap.add_argument("--showbus", action="store_true", help="PCIe generation and width")
    ap.add_argument("--showmodes", action="store_true", help="compute, persistence, MIG and ECC modes (read only)")
    ap.add_argument("--showtoponuma", action="store_true", help="NUMA node and local CPUs of every GPU")
    ap.add_argument("--showactivity", action="store_true", help="SM busy / occupancy / tensor / DRAM / FP activity and PCIe / NVLink traffic over 100 ms")
    ap.add_argument("--showevents", type=float, default=0.0, metavar="SECONDS",
                    help="print XID / ECC / power-state / clock events as they happen; stops after this long without one")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("-d", "--device", nargs="+", type=int, default=None, metavar="GPU", help="only these GPUs in the per-GPU listings (default: all)")
    for flag, help_ in (("--showserial", "serial and part number"), ("--showvbios", "VBIOS version"), ("--showfwinfo", "VBIOS and InfoROM image versions"),
                        ("--showperflevel", "performance state (P0 = fastest)"), ("--showmaxpower", "range the power limit can be set in"),
                        ("--showenergycounter", "energy drawn since the driver was loaded"), ("--showretiredpages", "rows of device memory remapped after errors")):
        ap.add_argument(flag, action="store_true", help=help_ + " (one line per GPU)")
    ap.add_argument("--setpowerlimit", nargs=2, metavar=("GPU", "WATTS"))
    ap.add_argument("--setclocks", nargs=3, metavar=("GPU", "MIN_MHZ", "MAX_MHZ"), help="lock the SM clock into a range (stays until --resetclocks)")
    ap.add_argument("--resetclocks", metavar="GPU", help="hand the SM clock back to the driver")
    ap.add_argument("--allow-set", action="store_true", help="required (with B200SMI_ALLOW_SET=1) before any setter acts")
    a = ap.parse_args(argv)
    try:
        smi = Smi()
    except RuntimeError as e:
        print(f"b200-smi: {e}", file=sys.stderr)
        return 1
    n = smi.count()
    devs = list(range(n)) if a.device is None else list(a.device)
    if any(not 0 <= d < n for d in devs):
        print(f"b200-smi: no GPU {next(d for d in devs if not 0 <= d < n)} (there are {n})", file=sys.stderr)
        return 2
    out = {}
    if a.setpowerlimit:
        try:
            smi.set_power_limit(int(a.setpowerlimit[0]), int(float(a.setpowerlimit[1]) * 1000), a.allow_set)
            print(f"power limit of GPU {a.setpowerlimit[0]} set to {a.setpowerlimit[1]} W")
        except RuntimeError as e:
            print(f"b200-smi: {e}", file=sys.stderr)
            return 2
    for what, act in (("setclocks", lambda v: smi.set_locked_clocks(int(v[0]), int(v[1]), int(v[2]), a.allow_set)),
                      ("resetclocks", lambda v: smi.reset_locked_clocks(int(v), a.allow_set))):
        v = getattr(a, what)
        if v:
            try:
                act(v)
                print(f"{what}: done for GPU {v[0] if isinstance(v, list) else v}")
            except RuntimeError as e:
                print(f"b200-smi: {e}", file=sys.stderr)
                return 2
    if a.showdriverversion or a.showall:
        out["driver_version"] = smi.driver_version()
        if not a.json:
            print(f"Driver version: {out['driver_version']}")
    if a.showpids:
        out["processes"] = {i: smi.processes(i) for i in devs}
        if not a.json:
            print(f"{'GPU':<4}{'PID':<10}{'Memory GiB':<12}Name")
            for i, ps in out["processes"].items():
                for pr in ps:
                    print(f"{i:<4}{pr['pid']:<10}{pr['used_memory_bytes'] / 2**30:<12.2f}{pr['name']}")
    if a.shownvlinkerrors:
        out["nvlink_errors"] = [smi.nvlink_errors(i) for i in devs]
        if not a.json:
            print(f"{'GPU':<4}{'links':<7}{'replay':<10}{'recovery':<10}{'crc flit':<10}{'crc data':<10}")
            for i, e in zip(devs, out["nvlink_errors"]):
                print(f"{i:<4}{e['linksRead']:<7}{e['replay']:<10}{e['recovery']:<10}{e['crcFlit']:<10}{e['crcData']:<10}")
    if a.showbus:
        out["pcie"] = [smi.pcie(i) for i in devs]
        if not a.json:
            for i, e in zip(devs, out["pcie"]):
                print(f"GPU{i}: PCIe gen {e['generation']} x{e['width']}")
    if a.showmodes:
        out["modes"] = [smi.modes(i) for i in devs]
        if not a.json:
            for i, m in zip(devs, out["modes"]):
                print(f"GPU{i}: compute mode {m['compute_mode']}, persistence {m['persistence']}, MIG {m['mig']}, ECC {m['ecc']}")
    id_flags = {"showserial": lambda d: f"serial {d['serial'] or 'n/a'}, part number {d['part_number'] or 'n/a'}", "showvbios": lambda d: f"VBIOS {d['vbios'] or 'n/a'}",
                "showfwinfo": lambda d: f"VBIOS {d['vbios'] or 'n/a'}, InfoROM image {d['inforom_image'] or 'n/a'}",
                "showperflevel": lambda d: "n/a" if d["performance_state"] is None else f"P{d['performance_state']}",
                "showmaxpower": lambda d: "n/a" if d["power_limit_max_w"] is None else f"power limit settable in {d['power_limit_min_w']:.0f} - {d['power_limit_max_w']:.0f} W",
                "showenergycounter": lambda d: "n/a" if d["energy_j"] is None else f"{d['energy_j']:.1f} J since the driver was loaded",
                "showretiredpages": lambda d: "n/a" if d["remapped_rows"] is None else
                f"remapped rows: {d['remapped_rows']['correctable']} correctable, {d['remapped_rows']['uncorrectable']} uncorrectable"
                f"{', remap pending' if d['remapped_rows']['pending'] else ''}{', REMAP FAILED' if d['remapped_rows']['failed'] else ''}"}
    id_asked = [k for k in id_flags if getattr(a, k)]
    if id_asked:
        out["identity"] = [smi.identity(i) for i in devs]
        if not a.json:
            for i, d in zip(devs, out["identity"]):
                print(f"GPU{i}: " + "; ".join(id_flags[k](d) for k in id_asked))
    if a.showtoponuma:
        from ..utils.affinity import format_cpu_list

        out["numa"] = [smi.cpu_affinity(i) for i in devs]
        if not a.json:
            for i, v in zip(devs, out["numa"]):
                print(f"GPU{i}: NUMA node {'n/a' if v['numa_node'] is None else v['numa_node']}, CPUs {format_cpu_list(v['cpus']) or 'n/a'}")
    if a.showactivity:
        out["activity"] = [smi.activity(i) for i in devs]
        if not a.json:
            fmt = lambda v, unit: "n/a" if v is None else f"{v:g}{unit}"  # noqa: E731
            for i, v in zip(devs, out["activity"]):
                print(f"GPU{i}: SM busy {fmt(v['sm_active_pct'], ' %')}, occupancy {fmt(v['sm_occupancy_pct'], ' %')}, tensor {fmt(v['tensor_active_pct'], ' %')}, "
                      f"DRAM {fmt(v['dram_active_pct'], ' %')}, fp64/32/16 {fmt(v['fp64_active_pct'], '')}/{fmt(v['fp32_active_pct'], '')}/{fmt(v['fp16_active_pct'], '')} %, "
                      f"PCIe tx/rx {fmt(v['pcie_tx_mibs'], '')}/{fmt(v['pcie_rx_mibs'], '')} MiB/s, NVLink tx/rx {fmt(v['nvlink_tx_mibs'], '')}/{fmt(v['nvlink_rx_mibs'], '')} MiB/s "
                      f"(over {v['interval_ms']:.0f} ms)")
    if a.showevents > 0:
        out["events"] = []
        for ev in smi.events(timeout_ms=int(a.showevents * 1000)):
            out["events"].append(ev)
            if not a.json:
                print(f"GPU{ev['device']}: {ev['type']} data={ev['data']} at {ev['timestamp_ns']}", flush=True)
    singles = {"showtemp": lambda d: f"{d['temperatureC']} C", "showpower": lambda d: f"{d['powerMilliwatt'] / 1000:.1f} W (limit {d['powerLimitMilliwatt'] / 1000:.0f} W)",
               "showclocks": lambda d: f"SM {d['smClockMhz']}/{d['smClockMaxMhz']} MHz, memory {d['memClockMhz']}/{d['memClockMaxMhz']} MHz",
               "showmeminfo": lambda d: f"{d['memUsedBytes'] / 2**30:.1f} / {d['memTotalBytes'] / 2**30:.1f} GiB", "showuse": lambda d: f"GPU {d['gpuUtilPct']} %, memory {d['memUtilPct']} %",
               "showuniqueid": lambda d: d["uuid"], "showproductname": lambda d: d["name"],
               "showecc": lambda d: f"corrected {d['eccCorrected']}, uncorrected {d['eccUncorrected']}",
               "showthrottle": lambda d: ",".join(d["throttleReasonNames"]) or "-"}
    asked = [k for k in singles if getattr(a, k)]
    if asked:
        infos = [smi.info(i) for i in devs]
        out["devices"] = infos
        if not a.json:
            for i, d in zip(devs, infos):
                print(f"GPU{i}: " + "; ".join(singles[k](d) for k in asked))
    only_new = bool(asked) or a.showtoponuma or bool(id_asked) or bool(a.setclocks) or bool(a.resetclocks) or a.showevents > 0 or a.showactivity or a.showmodes or a.showpids or a.shownvlinkerrors or a.showbus or a.showdriverversion
    tables = [("weight", "Weight between two GPUs", a.showtopoweight), ("hops", "Hops between two GPUs", a.showtopohops),
              ("typeName", "Link type between two GPUs", a.showtopotype), ("maxBandwidthMBps", "Max bandwidth (MB/s per direction)", a.shownodesbw),
              ("p2pAccessible", "Peer access between two GPUs", a.showtopoaccess)]
    one_table = any(t[2] for t in tables)
    if a.showall or not (a.showtopo or one_table or a.showhealth or a.setpowerlimit or only_new):
        out["devices"] = [smi.info(i) for i in devs]
        if not a.json:
            print(f"{'GPU':<4}{'Name':<22}{'Bus':<18}{'SM MHz':<12}{'Power W':<10}{'Temp C':<8}{'Mem used/total GiB':<22}{'NVLink':<8}{'Throttle'}")
            for i, d in zip(devs, out["devices"]):
                print(f"{i:<4}{d['name'][:20]:<22}{d['busId']:<18}{str(d['smClockMhz']) + '/' + str(d['smClockMaxMhz']):<12}{d['powerMilliwatt'] / 1000:<10.1f}"
                      f"{d['temperatureC']:<8}{d['memUsedBytes'] / 2**30:>6.1f} / {d['memTotalBytes'] / 2**30:<11.1f}{str(d['nvlinkActive']) + '/' + str(d['nvlinkCount']):<8}"
                      f"{','.join(d['throttleReasonNames']) or '-'}")
    if a.showtopo:
        out["topology"] = {k: _matrix(smi, k, n) for k in ("weight", "hops", "typeName", "maxBandwidthMBps", "p2pAccessible", "atomics64")}
        if not a.json:
            _print_matrix("Weight between two GPUs", out["topology"]["weight"], n)
            _print_matrix("Hops between two GPUs", out["topology"]["hops"], n)
            _print_matrix("Link type between two GPUs", out["topology"]["typeName"], n)
            _print_matrix("Max bandwidth (MB/s per direction)", out["topology"]["maxBandwidthMBps"], n)
    if one_table and not a.showtopo:
        out["topology"] = {k: _matrix(smi, k, n) for k, _, on in tables if on}
        if not a.json:
            for k, title, on in tables:
                if on:
                    _print_matrix(title, out["topology"][k], n)
    if a.showhealth:
        out["health"] = [dict(zip(("level", "reason"), smi.health(i))) for i in devs]
        if not a.json:
            for i, h in zip(devs, out["health"]):
                print(f"GPU{i}: {('PASS', 'WARN', 'FAIL')[h['level']]} - {h['reason']}")
    if a.json:
        print(json.dumps(out, indent=1))
    smi.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
