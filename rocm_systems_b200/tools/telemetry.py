"""Telemetry daemon and client: sample device fields in the background, keep a history, expose
them to Prometheus and over a small HTTP API, compute per-job statistics, report health.

The counterpart of the reference's data-center tool: the ``rdcd`` daemon, the ``rdci`` client
(rdc/rdci/src: discovery, dmon, group / field group, stats, diag) and its Prometheus plugin
(rdc/python_binding/rdc_prometheus.py). The sampling itself is native (``b200smi_watch_*`` in
csrc/core/health.cc, a sampler thread over NVML); this module is the service around it.

    python -m rocm_systems_b200.tools.telemetry serve --port 9400 --period-ms 1000
    curl localhost:9400/metrics
    python -m rocm_systems_b200.tools.telemetry discovery
    python -m rocm_systems_b200.tools.telemetry dmon -c 5 -d 1000 -e sm_clock power temp
    python -m rocm_systems_b200.tools.telemetry client --url http://127.0.0.1:9400 job-start --job run1
    python -m rocm_systems_b200.tools.telemetry client --url http://127.0.0.1:9400 job-stats --job run1

Nothing here changes a device setting.
"""
from __future__ import annotations

import argparse
import json
import sys
import threading
import time
import urllib.parse
import urllib.request
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import List, Optional, Sequence

from .smi import ACTIVITY_FIELDS, FIELDS, REASON_BITS, Smi

DEFAULT_FIELDS = ["sm_clock", "mem_clock", "power", "temp", "mem_used", "gpu_util", "mem_util", "ecc_corrected", "ecc_uncorrected",
                  "throttle_reasons", "nvlink_active"]
# field -> (metric name, help, scale to the metric's unit)
PROM = {
    "sm_clock": ("b200_sm_clock_mhz", "SM clock in MHz", 1.0),
    "mem_clock": ("b200_memory_clock_mhz", "memory clock in MHz", 1.0),
    "power": ("b200_power_watts", "board power draw in watts", 1.0),
    "temp": ("b200_temperature_celsius", "GPU temperature", 1.0),
    "mem_used": ("b200_memory_used_bytes", "device memory in use", 1.0),
    "gpu_util": ("b200_gpu_utilization_percent", "fraction of time a kernel was running", 1.0),
    "mem_util": ("b200_memory_utilization_percent", "fraction of time memory was read or written", 1.0),
    "ecc_corrected": ("b200_ecc_corrected_total", "corrected ECC errors (volatile)", 1.0),
    "ecc_uncorrected": ("b200_ecc_uncorrected_total", "uncorrected ECC errors (volatile)", 1.0),
    "throttle_reasons": ("b200_clock_event_reasons", "bit mask of active clock event reasons", 1.0),
    "nvlink_active": ("b200_nvlink_active_links", "NVLink links in the active state", 1.0),
    # activity over the sampling period (the field group "activity"; what the reference's profiler plug-in adds to its telemetry)
    "sm_active": ("b200_sm_active_percent", "share of SMs that were busy", 1.0),
    "sm_occupancy": ("b200_sm_occupancy_percent", "resident warps against the maximum", 1.0),
    "tensor_active": ("b200_tensor_active_percent", "share of time the tensor pipes were busy", 1.0),
    "dram_active": ("b200_dram_bandwidth_percent", "DRAM bandwidth used against the maximum", 1.0),
    "fp64_active": ("b200_fp64_active_percent", "share of time the FP64 pipes were busy", 1.0),
    "fp32_active": ("b200_fp32_active_percent", "share of time the FP32 pipes were busy", 1.0),
    "fp16_active": ("b200_fp16_active_percent", "share of time the FP16 pipes were busy", 1.0),
    "pcie_tx_mibs": ("b200_pcie_tx_bytes_per_second", "PCIe traffic from the GPU", 1048576.0),
    "pcie_rx_mibs": ("b200_pcie_rx_bytes_per_second", "PCIe traffic to the GPU", 1048576.0),
    "nvlink_tx_mibs": ("b200_nvlink_tx_bytes_per_second", "NVLink traffic from the GPU, all links", 1048576.0),
    "nvlink_rx_mibs": ("b200_nvlink_rx_bytes_per_second", "NVLink traffic to the GPU, all links", 1048576.0),
}


class Telemetry:
    """Field groups and device groups over the native watch, plus text renderings."""

    def __init__(self, smi: Optional[Smi] = None):
        self.smi = smi or Smi()
        self.devices: List[int] = list(range(self.smi.count()))
        self.fields: List[str] = list(DEFAULT_FIELDS)
        self.watching = False
        self.jobs: dict = {}
        self.groups: dict = {"all": list(self.devices)}          # device groups by name
        self.field_groups: dict = {"default": list(DEFAULT_FIELDS), "activity": list(ACTIVITY_FIELDS)}
        self.device_events: List[dict] = []                      # XID / ECC / clock events seen by the listener
        self._event_thread: Optional[threading.Thread] = None
        self._event_stop = threading.Event()

    # ---- groups (rdc: rdc_group_gpu_create / rdc_group_field_create / rdc_field_watch) ----
    def create_group(self, name: str, devices: Sequence[int]) -> None:
        n = self.smi.count()
        bad = [d for d in devices if not 0 <= d < n]
        if bad:
            raise ValueError(f"no such device(s) {bad}; this host has {n}")
        self.groups[name] = list(devices)

    def create_field_group(self, name: str, fields: Sequence[str]) -> None:
        unknown = [f for f in fields if f not in FIELDS]
        if unknown:
            raise ValueError(f"unknown field(s) {unknown}; known: {sorted(FIELDS)}")
        self.field_groups[name] = list(fields)

    def delete_group(self, name: str) -> None:
        if name == "all":
            raise ValueError("the group of all devices cannot be deleted")
        if name not in self.groups:
            raise KeyError(f"no device group {name!r}")
        del self.groups[name]

    def delete_field_group(self, name: str) -> None:
        if name == "default":
            raise ValueError("the default field group cannot be deleted")
        if name not in self.field_groups:
            raise KeyError(f"no field group {name!r}")
        del self.field_groups[name]

    def watch(self, group: str = "all", field_group: str = "default", period_ms: int = 1000, keep: int = 3600) -> None:
        if group not in self.groups:
            raise KeyError(f"no device group {group!r}")
        if field_group not in self.field_groups:
            raise KeyError(f"no field group {field_group!r}")
        if self.watching:
            self.stop()
        self.start(self.groups[group], self.field_groups[field_group], period_ms, keep)

    def topology(self, dev: int) -> List[dict]:
        """The links of ``dev`` to every other device (rdc: rdc_device_topology_get)."""
        n = self.smi.count()
        if not 0 <= dev < n:
            raise ValueError(f"no device {dev}; this host has {n}")
        out = []
        for peer in range(n):
            if peer != dev:
                l = self.smi.link(dev, peer)
                out.append({"peer": peer, "type": l["typeName"], "hops": l["hops"], "weight": l["weight"], "max_bandwidth_mbps": l["maxBandwidthMBps"],
                            "peer_access": bool(l["p2pAccessible"])})
        return out

    # ---- settings that outlive the daemon (rdc: RdcConfigSettingsImpl: groups, field groups and policies kept in a file) ----
    def config(self) -> dict:
        return {"groups": {k: v for k, v in self.groups.items() if k != "all"}, "field_groups": {k: v for k, v in self.field_groups.items() if k != "default"},
                "policies": list(getattr(self, "_policies", []))}

    def config_save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.config(), f, indent=1)

    def config_load(self, path: str) -> dict:
        """Re-creates the groups, field groups and policies of a saved file; entries that do not fit this host (a device
        index that is not there, an unknown field) are reported and skipped, the rest is applied."""
        with open(path) as f:
            cfg = json.load(f)
        skipped = []
        for name, devs in cfg.get("groups", {}).items():
            try:
                self.create_group(name, devs)
            except ValueError as e:
                skipped.append(f"group {name}: {e}")
        for name, fields in cfg.get("field_groups", {}).items():
            try:
                self.create_field_group(name, fields)
            except ValueError as e:
                skipped.append(f"field group {name}: {e}")
        for p in cfg.get("policies", []):
            try:
                self.policy_set(int(p["device"]), p["field"], float(p["threshold"]), p.get("direction", "above") != "below")
            except (ValueError, KeyError, RuntimeError) as e:
                skipped.append(f"policy {p}: {e}")
        return {"applied": self.config(), "skipped": skipped}

    def diagnose(self, level: int = 1) -> List[dict]:
        """Short diagnostics per device (rdc: rdc_diagnostic_run). Level 1 reads only: health verdict,
        every link up, no uncorrected ECC, no link errors, PCIe link trained at full width. Level 2
        adds a device-memory bandwidth check when this process can use CUDA."""
        out = []
        for d in self.devices:
            checks = []
            lvl, msg = self.smi.health(d)
            checks.append({"check": "health", "pass": lvl == 0, "detail": msg})
            i = self.smi.info(d)
            checks.append({"check": "nvlink_up", "pass": i["nvlinkActive"] == i["nvlinkCount"], "detail": f"{i['nvlinkActive']}/{i['nvlinkCount']} links"})
            checks.append({"check": "ecc_uncorrected", "pass": i["eccUncorrected"] == 0, "detail": str(i["eccUncorrected"])})
            try:
                e = self.smi.nvlink_errors(d)
                bad = e["replay"] + e["recovery"] + e["crcFlit"] + e["crcData"]
                checks.append({"check": "nvlink_errors", "pass": bad == 0, "detail": json.dumps(e)})
                pc = self.smi.pcie(d)
                checks.append({"check": "pcie_link", "pass": pc["width"] >= 16, "detail": f"gen {pc['generation']} x{pc['width']}"})
            except RuntimeError as err:
                checks.append({"check": "nvlink_errors", "pass": True, "detail": f"not available: {err}"})
            if level >= 2:
                checks.append(self._bandwidth_check(d))
            out.append({"device": d, "pass": all(c["pass"] for c in checks), "checks": checks})
        return out

    @staticmethod
    def _bandwidth_check(dev: int, nbytes: int = 1 << 30, floor_gbs: float = 3000.0) -> dict:
        try:
            import torch

            if not torch.cuda.is_available() or dev >= torch.cuda.device_count():
                return {"check": "memory_bandwidth", "pass": True, "detail": "skipped: CUDA not usable from this process"}
            with torch.cuda.device(dev):
                a = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
                b = torch.empty_like(a)
                for _ in range(2):
                    b.copy_(a)
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for _ in range(5):
                    b.copy_(a)
                e.record()
                torch.cuda.synchronize()
                gbs = 2 * nbytes * 5 / (s.elapsed_time(e) * 1e-3) / 1e9
            return {"check": "memory_bandwidth", "pass": gbs >= floor_gbs, "detail": f"{gbs:.0f} GB/s copy (floor {floor_gbs:.0f})"}
        except Exception as err:  # noqa: BLE001 - a diagnostic reports, it does not raise
            return {"check": "memory_bandwidth", "pass": False, "detail": str(err)}

    def start(self, devices: Optional[Sequence[int]] = None, fields: Optional[Sequence[str]] = None, period_ms: int = 1000, keep: int = 3600) -> None:
        if devices is not None:
            self.devices = list(devices)
        if fields is not None:
            unknown = [f for f in fields if f not in FIELDS]
            if unknown:
                raise ValueError(f"unknown field(s) {unknown}; known: {sorted(FIELDS)}")
            self.fields = list(fields)
        self.smi.watch_start(self.devices, self.fields, period_ms, keep)
        self.watching = True

    def stop(self) -> None:
        if self.watching:
            self.smi.watch_stop()
            self.watching = False
        self.stop_event_listener()

    # ---- asynchronous device events (rdc notifications / rsmi_event_notification_*) ----
    def start_event_listener(self, keep: int = 1000) -> None:
        """A background thread that records XID errors, ECC errors and clock / power-state changes as they happen."""
        if self._event_thread is not None:
            return
        self._event_stop.clear()

        def run() -> None:
            try:
                for ev in self.smi.events(timeout_ms=200, stop=self._event_stop):
                    self.device_events.append(ev)
                    del self.device_events[:-keep]
                    if self._event_stop.is_set():
                        break
            except RuntimeError:  # the driver has no event support: nothing to listen to
                return

        self._event_thread = threading.Thread(target=run, daemon=True)
        self._event_thread.start()

    def stop_event_listener(self) -> None:
        if self._event_thread is not None:
            self._event_stop.set()
            self._event_thread.join(timeout=2)
            self._event_thread = None

    def discovery(self) -> List[dict]:
        out = []
        for d in range(self.smi.count()):
            i = self.smi.info(d)
            out.append({"index": d, "name": i["name"], "uuid": i["uuid"], "bus_id": i["busId"], "memory_total_bytes": i["memTotalBytes"],
                        "nvlinks": i["nvlinkCount"], "multicast_capable": bool(i["multicastCapable"])})
        return out

    def latest(self) -> dict:
        """{device: {field: value}} read now (not from the history); ``None`` for a field this device does not report."""
        def read(d, f):
            try:
                return self.smi.read(d, f)
            except RuntimeError as e:
                if "not supported" in str(e):
                    return None
                raise

        return {d: {f: read(d, f) for f in self.fields} for d in self.devices}

    def history(self, dev: int, field: str, max_n: int = 4096) -> list:
        return self.smi.history(dev, field, max_n)

    def job_start(self, job: str) -> None:
        self.smi.job_start(job)
        self.jobs[job] = {"start": time.time(), "stop": None}

    def job_stop(self, job: str) -> None:
        self.smi.job_stop(job)
        if job in self.jobs:
            self.jobs[job]["stop"] = time.time()

    # ---- policies (rdc: rdc_policy_set / rdc_policy_register: a threshold on a field fires a notification) ----
    def policy_set(self, dev: int, field: str, threshold: float, above: bool = True) -> None:
        """Record an event whenever ``field`` of ``dev`` crosses ``threshold`` while it is being watched.
        Events accumulate in ``policy_events()``; nothing is done to the device."""
        if field not in FIELDS:
            raise ValueError(f"unknown field {field!r}; known: {sorted(FIELDS)}")
        if not hasattr(self, "_events"):
            self._events = []
            self._events_lock = threading.Lock()
        names = {v: k for k, v in FIELDS.items()}

        def fire(d, f, value, thr):
            with self._events_lock:
                self._events.append({"time": time.time(), "device": d, "field": names.get(f, str(f)), "value": value, "threshold": thr,
                                     "direction": "above" if above else "below"})
                del self._events[:-1000]  # keep the last thousand

        self.smi.policy(dev, field, threshold, above, fire)
        if not hasattr(self, "_policies"):
            self._policies = []
        self._policies = [p for p in self._policies if not (p["device"] == dev and p["field"] == field and p["direction"] == ("above" if above else "below"))]
        self._policies.append({"device": dev, "field": field, "threshold": threshold, "direction": "above" if above else "below"})

    def policy_events(self) -> list:
        if not hasattr(self, "_events"):
            return []
        with self._events_lock:
            return list(self._events)

    def job_stats(self, job: str) -> dict:
        out = {"job": job, **self.jobs.get(job, {}), "devices": {}}
        for d in self.devices:
            out["devices"][d] = {f: self.smi.job_stats(job, d, f) for f in self.fields}
        return out

    def health(self) -> dict:
        names = {0: "PASS", 1: "WARN", 2: "FAIL"}
        out = {}
        for d in self.devices:
            level, msg = self.smi.health(d)
            out[d] = {"level": names.get(level, str(level)), "message": msg}
        return out

    def prometheus(self) -> str:
        vals = self.latest()
        infos = {d: self.smi.info(d) for d in self.devices}
        lines = []
        for f in self.fields:
            name, help_, scale = PROM[f]
            kind = "counter" if name.endswith("_total") else "gauge"
            lines.append(f"# HELP {name} {help_}")
            lines.append(f"# TYPE {name} {kind}")
            for d in self.devices:
                if vals[d][f] is not None:
                    lines.append(f'{name}{{gpu="{d}",uuid="{infos[d]["uuid"]}"}} {vals[d][f] * scale:.12g}')
        if "throttle_reasons" in self.fields:
            lines.append("# HELP b200_clock_event_reason one series per reason; 1 while it is active")
            lines.append("# TYPE b200_clock_event_reason gauge")
            for d in self.devices:
                mask = int(vals[d]["throttle_reasons"] or 0)
                for bit, reason in REASON_BITS.items():
                    lines.append(f'b200_clock_event_reason{{gpu="{d}",reason="{reason}"}} {1 if mask & bit else 0}')
        try:  # link error counters, where the driver exposes them
            errs = {d: self.smi.nvlink_errors(d) for d in self.devices}
            for key, metric in (("replay", "b200_nvlink_replay_errors_total"), ("recovery", "b200_nvlink_recovery_errors_total"),
                                ("crcFlit", "b200_nvlink_crc_flit_errors_total"), ("crcData", "b200_nvlink_crc_data_errors_total")):
                lines.append(f"# HELP {metric} NVLink {key} errors summed over the device's links")
                lines.append(f"# TYPE {metric} counter")
                for d in self.devices:
                    lines.append(f'{metric}{{gpu="{d}"}} {errs[d][key]}')
        except RuntimeError:
            pass
        if self.device_events:
            lines.append("# HELP b200_device_events_total asynchronous device events seen since the listener started")
            lines.append("# TYPE b200_device_events_total counter")
            counts: dict = {}
            for ev in self.device_events:
                counts[(ev["device"], ev["type"])] = counts.get((ev["device"], ev["type"]), 0) + 1
            for (d, kind), c in sorted(counts.items()):
                lines.append(f'b200_device_events_total{{gpu="{d}",type="{kind}"}} {c}')
        return "\n".join(lines) + "\n"


def make_handler(t: Telemetry):
    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *args) -> None:  # quiet
            pass

        def _send(self, code: int, body: str, ctype: str = "application/json") -> None:
            data = body.encode()
            self.send_response(code)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def do_GET(self) -> None:  # noqa: N802 - name fixed by the base class
            url = urllib.parse.urlparse(self.path)
            q = {k: v[0] for k, v in urllib.parse.parse_qs(url.query).items()}
            try:
                if url.path == "/metrics":
                    self._send(200, t.prometheus(), "text/plain; version=0.0.4")
                elif url.path == "/api/devices":
                    self._send(200, json.dumps(t.discovery()))
                elif url.path == "/api/latest":
                    self._send(200, json.dumps(t.latest()))
                elif url.path == "/api/history":
                    self._send(200, json.dumps(t.history(int(q["dev"]), q["field"], int(q.get("max", 4096)))))
                elif url.path == "/api/health":
                    self._send(200, json.dumps(t.health()))
                elif url.path == "/api/job/start":
                    t.job_start(q["job"])
                    self._send(200, json.dumps({"ok": True}))
                elif url.path == "/api/job/stop":
                    t.job_stop(q["job"])
                    self._send(200, json.dumps({"ok": True}))
                elif url.path == "/api/job/stats":
                    self._send(200, json.dumps(t.job_stats(q["job"])))
                elif url.path == "/api/policy/set":
                    t.policy_set(int(q["dev"]), q["field"], float(q["threshold"]), q.get("direction", "above") != "below")
                    self._send(200, json.dumps({"ok": True}))
                elif url.path == "/api/policy/list":
                    self._send(200, json.dumps(list(getattr(t, "_policies", []))))
                elif url.path == "/api/group/create":
                    t.create_group(q["name"], [int(x) for x in q["devices"].split(",") if x != ""])
                    self._send(200, json.dumps({"ok": True}))
                elif url.path == "/api/group/delete":
                    t.delete_group(q["name"])
                    self._send(200, json.dumps({"ok": True}))
                elif url.path == "/api/group/list":
                    self._send(200, json.dumps(t.groups))
                elif url.path == "/api/fieldgroup/create":
                    t.create_field_group(q["name"], [x for x in q["fields"].split(",") if x])
                    self._send(200, json.dumps({"ok": True}))
                elif url.path == "/api/fieldgroup/delete":
                    t.delete_field_group(q["name"])
                    self._send(200, json.dumps({"ok": True}))
                elif url.path == "/api/fieldgroup/list":
                    self._send(200, json.dumps(t.field_groups))
                elif url.path == "/api/watch":
                    t.watch(q.get("group", "all"), q.get("fieldgroup", "default"), int(q.get("period_ms", 1000)), int(q.get("keep", 3600)))
                    self._send(200, json.dumps({"ok": True, "devices": t.devices, "fields": t.fields}))
                elif url.path == "/api/topo":
                    self._send(200, json.dumps(t.topology(int(q.get("dev", 0)))))
                elif url.path == "/api/config":
                    self._send(200, json.dumps(t.config()))
                elif url.path == "/api/config/save":
                    t.config_save(q["path"])
                    self._send(200, json.dumps({"ok": True}))
                elif url.path == "/api/config/load":
                    self._send(200, json.dumps(t.config_load(q["path"])))
                elif url.path == "/api/events":
                    self._send(200, json.dumps(t.device_events))
                elif url.path == "/api/policy/events":
                    self._send(200, json.dumps(t.policy_events()))
                else:
                    self._send(404, json.dumps({"error": "unknown path"}))
            except (KeyError, ValueError, RuntimeError, OSError) as e:
                self._send(400, json.dumps({"error": str(e)}))

    return Handler


def serve(t: Telemetry, host: str, port: int) -> ThreadingHTTPServer:
    """Starts the HTTP server on a thread and returns it (``shutdown()`` stops it)."""
    srv = ThreadingHTTPServer((host, port), make_handler(t))
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv


def _client(url: str, endpoint: str, **q) -> object:
    path = endpoint
    full = url.rstrip("/") + path + ("?" + urllib.parse.urlencode(q) if q else "")
    with urllib.request.urlopen(full, timeout=10) as r:
        body = r.read().decode()
    return body if path == "/metrics" else json.loads(body)


class Reader:
    """Periodic reader for programs that want the values themselves (a logger, a scheduler, a plug-in of another monitoring
    system): subclass it and override ``handle_field``, or pass ``on_field``. Embedded (its own ``Telemetry`` in this
    process) when ``url`` is None, else a client of a running daemon. The reference ships the same helper for its daemon
    (rdc/python_binding/RdcReader.py: ``RdcReader(ip_port, field_ids, update_freq, ...)`` with ``process()`` calling
    ``handle_field(gpu_index, value)``), and builds its Prometheus and collectd plug-ins on it.

        class Log(Reader):
            def handle_field(self, device, field, value, timestamp_ns): print(device, field, value)
        Log(fields=["power", "tensor_active"], period_ms=500).run(iterations=10)
    """

    def __init__(self, url: Optional[str] = None, fields: Optional[Sequence[str]] = None, devices: Optional[Sequence[int]] = None, period_ms: int = 1000,
                 on_field=None, telemetry: Optional[Telemetry] = None):
        self.url = url
        self.fields = list(fields or DEFAULT_FIELDS)
        unknown = [f for f in self.fields if f not in FIELDS]
        if unknown:
            raise ValueError(f"unknown field(s) {unknown}; known: {', '.join(FIELDS)}")
        self.period_ms = period_ms
        self.on_field = on_field
        self.t = None
        if url is None:
            self.t = telemetry or Telemetry()
            self.t.fields = list(self.fields)
            self.devices = list(devices) if devices is not None else list(self.t.devices)
            self.t.devices = list(self.devices)
        else:
            known = [d["index"] if isinstance(d, dict) and "index" in d else i for i, d in enumerate(_client(url, "/api/devices"))]
            self.devices = list(devices) if devices is not None else known
        self.reads = 0

    def handle_field(self, device: int, field: str, value: Optional[float], timestamp_ns: int) -> None:
        if self.on_field:
            self.on_field(device, field, value, timestamp_ns)

    def process(self) -> int:
        """One round: every (device, field) once; returns how many values were handed over (unsupported ones are skipped)."""
        now = time.time_ns()
        if self.t is not None:
            latest = self.t.latest()
        else:
            latest = {int(k): v for k, v in _client(self.url, "/api/latest").items()}
        n = 0
        for d in self.devices:
            for f in self.fields:
                v = latest.get(d, {}).get(f)
                if v is not None:
                    self.handle_field(d, f, v, now)
                    n += 1
        self.reads += 1
        return n

    def run(self, iterations: int = 0, stop: Optional[threading.Event] = None) -> None:
        """Calls ``process`` every period until ``iterations`` rounds are done (0: until ``stop`` is set)."""
        i = 0
        while (iterations == 0 or i < iterations) and not (stop and stop.is_set()):
            t0 = time.monotonic()
            self.process()
            i += 1
            if iterations == 0 or i < iterations:
                left = self.period_ms / 1000.0 - (time.monotonic() - t0)
                if left > 0:
                    (stop.wait(left) if stop else time.sleep(left))


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="telemetry", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("serve", help="run the daemon")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=9400)
    p.add_argument("--period-ms", type=int, default=1000)
    p.add_argument("--keep", type=int, default=3600, help="samples kept per device and field")
    p.add_argument("-e", "--fields", nargs="+", default=DEFAULT_FIELDS)
    p.add_argument("-i", "--devices", nargs="+", type=int)
    p.add_argument("--duration", type=float, default=0.0, help="exit after this many seconds (0 = run until interrupted)")
    sub.add_parser("discovery", help="list devices")
    p = sub.add_parser("dmon", help="print readings periodically")
    p.add_argument("-c", "--count", type=int, default=0)
    p.add_argument("-d", "--delay-ms", type=int, default=1000)
    p.add_argument("-e", "--fields", nargs="+", default=["sm_clock", "power", "temp", "gpu_util", "mem_used"])
    p.add_argument("-f", "--fieldgroup", default="", help="a field group instead of -e: default, activity")
    p.add_argument("-i", "--devices", nargs="+", type=int)
    p.add_argument("-l", "--list-fields", action="store_true", help="list the fields and field groups that can be watched and stop")
    sub.add_parser("health", help="one health verdict per device")
    p = sub.add_parser("diag", help="short diagnostics per device")
    p.add_argument("--level", type=int, default=1, choices=[1, 2])
    p = sub.add_parser("client", help="talk to a running daemon")
    p.add_argument("--url", default="http://127.0.0.1:9400")
    p.add_argument("what", choices=["devices", "latest", "health", "metrics", "history", "events", "job-start", "job-stop", "job-stats",
                                    "group-create", "group-delete", "group-list", "fieldgroup-create", "fieldgroup-delete", "fieldgroup-list", "watch",
                                    "policy-set", "policy-list", "policy-events", "topo", "config", "config-save", "config-load"])
    p.add_argument("--job", default="")
    p.add_argument("--dev", type=int, default=0)
    p.add_argument("--field", default="power")
    p.add_argument("--name", default="", help="group or field group")
    p.add_argument("--devices", nargs="+", type=int, default=[], help="group-create: device indices")
    p.add_argument("--fields", nargs="+", default=[], help="fieldgroup-create: field names")
    p.add_argument("--group", default="all", help="watch: device group")
    p.add_argument("--fieldgroup", default="default", help="watch: field group")
    p.add_argument("--period-ms", type=int, default=1000, help="watch: sampling period")
    p.add_argument("--threshold", type=float, default=0.0, help="policy-set")
    p.add_argument("--direction", choices=["above", "below"], default="above", help="policy-set")
    p.add_argument("--path", default="", help="config-save / config-load: file on the daemon's host")
    a = ap.parse_args(argv)

    if a.cmd == "client":
        path = {"devices": "/api/devices", "latest": "/api/latest", "health": "/api/health", "metrics": "/metrics", "history": "/api/history", "events": "/api/events",
                "job-start": "/api/job/start", "job-stop": "/api/job/stop", "job-stats": "/api/job/stats",
                "group-create": "/api/group/create", "group-delete": "/api/group/delete", "group-list": "/api/group/list",
                "fieldgroup-create": "/api/fieldgroup/create", "fieldgroup-delete": "/api/fieldgroup/delete", "fieldgroup-list": "/api/fieldgroup/list",
                "watch": "/api/watch", "policy-set": "/api/policy/set", "policy-list": "/api/policy/list", "policy-events": "/api/policy/events",
                "topo": "/api/topo", "config": "/api/config", "config-save": "/api/config/save", "config-load": "/api/config/load"}[a.what]
        q = {}
        if a.what.startswith("job"):
            q["job"] = a.job
        if a.what == "history":
            q = {"dev": a.dev, "field": a.field}
        if a.what == "group-create":
            q = {"name": a.name, "devices": ",".join(str(d) for d in a.devices)}
        if a.what == "fieldgroup-create":
            q = {"name": a.name, "fields": ",".join(a.fields)}
        if a.what in ("group-delete", "fieldgroup-delete"):
            q = {"name": a.name}
        if a.what == "watch":
            q = {"group": a.group, "fieldgroup": a.fieldgroup, "period_ms": a.period_ms}
        if a.what == "policy-set":
            q = {"dev": a.dev, "field": a.field, "threshold": a.threshold, "direction": a.direction}
        if a.what == "topo":
            q = {"dev": a.dev}
        if a.what in ("config-save", "config-load"):
            q = {"path": a.path}
        res = _client(a.url, path, **q)
        print(res if isinstance(res, str) else json.dumps(res, indent=1))
        return 0

    t = Telemetry()
    if a.cmd == "discovery":
        for d in t.discovery():
            print(f"{d['index']}\t{d['name']}\t{d['uuid']}\t{d['bus_id']}\t{d['memory_total_bytes'] / 2**30:.0f} GiB\tNVLink x{d['nvlinks']}")
    elif a.cmd == "health":
        for d, h in t.health().items():
            print(f"GPU {d}: {h['level']} {h['message']}")
    elif a.cmd == "diag":
        res = t.diagnose(a.level)
        for r in res:
            print(f"GPU {r['device']}: {'PASS' if r['pass'] else 'FAIL'}")
            for c in r["checks"]:
                print(f"    {c['check']:<18} {'ok' if c['pass'] else 'FAILED':<7} {c['detail']}")
        return 0 if all(r["pass"] for r in res) else 1
    elif a.cmd == "dmon":
        if a.list_fields:
            for f in FIELDS:
                print(f"{f:<18} {PROM[f][1] if f in PROM else ''}")
            for name, members in t.field_groups.items():
                print(f"group {name}: {' '.join(members)}")
            return 0
        if a.fieldgroup:
            if a.fieldgroup not in t.field_groups:
                print(f"telemetry: no field group {a.fieldgroup!r}; known: {', '.join(t.field_groups)}", file=sys.stderr)
                return 2
            a.fields = list(t.field_groups[a.fieldgroup])
        unknown = [f for f in a.fields if f not in FIELDS]
        if unknown:
            print(f"telemetry: unknown field(s) {unknown}; `dmon -l` lists them", file=sys.stderr)
            return 2
        t.fields = a.fields
        if a.devices:
            t.devices = a.devices
        print("GPU\t" + "\t".join(a.fields))
        n = 0
        while a.count == 0 or n < a.count:
            for d, vals in t.latest().items():
                print(f"{d}\t" + "\t".join("n/a" if vals[f] is None else f"{vals[f]:g}" for f in a.fields), flush=True)
            n += 1
            if a.count == 0 or n < a.count:
                time.sleep(a.delay_ms / 1e3)
    elif a.cmd == "serve":
        t.start(a.devices, a.fields, a.period_ms, a.keep)
        t.start_event_listener()
        srv = serve(t, a.host, a.port)
        print(f"telemetry: serving http://{a.host}:{srv.server_address[1]}/metrics for {len(t.devices)} device(s)", flush=True)
        try:
            if a.duration > 0:
                time.sleep(a.duration)
            else:
                while True:
                    time.sleep(3600)
        except KeyboardInterrupt:
            pass
        srv.shutdown()
        t.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
