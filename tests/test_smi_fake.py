"""b200smi against a fake NVML (no GPU): readings, topology table, watches, job statistics,
policies, health and the guarded setter. The reference tests rocm-smi against overridden sysfs
trees the same way (rocm-smi-lib/src/rocm_smi_main.cc:522-527)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def fake_nvml(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake_nvml") / "libfake_nvml.so"
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-o", str(out), str(ROOT / "tests" / "fake_nvml" / "fake_nvml.c")])
    return str(out)


def _run(code: str, fake: str, env=None):
    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake, PYTHONPATH=str(ROOT))
    e.update(env or {})
    p = subprocess.run([sys.executable, "-c", code], env=e, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr
    return p.stdout


def test_readings_and_topology(fake_nvml):
    out = _run("""
from rocm_systems_b200.tools.smi import Smi
s = Smi()
assert s.count() == 8
i = s.info(3)
assert i['name'].startswith('NVIDIA B200') and i['nvlinkCount'] == 18 and i['nvlinkActive'] == 18
assert i['smClockMaxMhz'] == 1965 and 'sw_power_cap' in i['throttleReasonNames']
l = s.link(0, 5)
assert l['typeName'] == 'NVLINK' and l['hops'] == 1 and l['weight'] == 15 and l['nvlinks'] == 18 and l['maxBandwidthMBps'] == 900000
assert s.link(2, 2)['typeName'] == 'SELF'
print('ok')
""", fake_nvml)
    assert "ok" in out


def test_cli_tables(fake_nvml):
    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake_nvml, PYTHONPATH=str(ROOT), FAKE_NVML_GPUS="4")
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "--showall", "--showtopo", "--showhealth"], env=e, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    assert "Weight between two GPUs" in p.stdout and "NVLINK" in p.stdout and "PASS" in p.stdout
    # one table at a time, as the reference CLI offers them (rocm_smi.py showWeightTopology / showHopsTopology / showTypeTopology / showNodesBw)
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "--showtopohops", "--shownodesbw"], env=e, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    assert "Hops between two GPUs" in p.stdout and "Max bandwidth" in p.stdout
    assert "Weight between two GPUs" not in p.stdout and "Name" not in p.stdout
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "--showtopoaccess", "--json"], env=e, capture_output=True, text=True)
    import json
    assert list(json.loads(p.stdout)["topology"]) == ["p2pAccessible"]


def test_health_flags_link_down_and_ecc(fake_nvml):
    out = _run("""
from rocm_systems_b200.tools.smi import Smi
s = Smi()
print(s.health(1)); print(s.health(2)); print(s.health(0))
assert s.link(1, 0)['nvlinks'] == 17
""", fake_nvml, {"FAKE_NVML_LINK_DOWN": "1", "FAKE_NVML_ECC": "2"})
    lines = out.strip().splitlines()
    assert lines[0].startswith("(2") and "17 of 18" in lines[0]
    assert lines[1].startswith("(2") and "uncorrected ECC" in lines[1]
    assert lines[2].startswith("(0")


def test_watch_job_stats_and_policy(fake_nvml):
    out = _run("""
import time
from rocm_systems_b200.tools.smi import Smi
s = Smi()
fired = []
s.policy(0, 'power', 260.0, True, lambda d, f, v, t: fired.append((d, v)))
s.job_start('job1')
s.watch_start([0, 1], ['power', 'temp'], period_ms=20, keep=50)
time.sleep(0.6)
s.job_stop('job1')
s.watch_stop()
h = s.history(0, 'power')
st = s.job_stats('job1', 0, 'power')
assert len(h) >= 5 and h[-1][1] > h[0][1]
assert st['samples'] >= 5 and st['max'] > st['min'] and st['min'] <= st['avg'] <= st['max']
assert fired and fired[0][0] == 0 and fired[0][1] > 260.0 and len(fired) == 1   # latched: fires once per excursion
print('ok')
""", fake_nvml, {"FAKE_NVML_RAMP": "1"})
    assert "ok" in out


def test_setter_is_off_by_default(fake_nvml):
    code = """
from rocm_systems_b200.tools.smi import Smi
s = Smi()
for allow in (False, True):
    try:
        s.set_power_limit(0, 700000, allow)
        print('set', allow)
    except RuntimeError as e:
        print('refused', allow)
print(s.info(0)['powerLimitMilliwatt'])
"""
    out = _run(code, fake_nvml).split()
    assert out == ["refused", "False", "refused", "True", "1000000"]          # env switch absent: nothing is written
    out = _run(code, fake_nvml, {"B200SMI_ALLOW_SET": "1"}).split()
    assert out == ["refused", "False", "set", "True", "700000"]               # only the fake GPU is ever touched


def test_driver_processes_link_errors_and_bus(fake_nvml):
    out = _run("""
import os
from rocm_systems_b200.tools.smi import Smi
s = Smi()
assert s.driver_version() == '580.159.fake'
ps = s.processes(0)
assert [p['pid'] for p in ps] == [os.getpid(), 1] and ps[0]['used_memory_bytes'] == 3 << 30 and ps[0]['name'].startswith('python')
assert s.processes(1) == []
e = s.nvlink_errors(2)
assert e['linksRead'] == 18 and e['replay'] == 5 and e['crcFlit'] == 0 and s.nvlink_errors(0)['replay'] == 0
assert s.pcie(3) == {'generation': 5, 'width': 16}
assert s.modes(1) == {'compute_mode': 'default', 'persistence': 1, 'mig': 0, 'ecc': 1}
print('ok')
""", fake_nvml, {"FAKE_NVML_LINK_ERRORS": "2"})
    assert "ok" in out
    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake_nvml, PYTHONPATH=str(ROOT), FAKE_NVML_GPUS="2")
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "--showpids", "--shownvlinkerrors", "--showbus", "--showdriverversion"],
                       env=e, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    assert "580.159.fake" in p.stdout and "PCIe gen 5 x16" in p.stdout and "Memory GiB" in p.stdout and "SM MHz" not in p.stdout


def test_event_stream(fake_nvml):
    """XID / ECC events come out of the event set in order with device index, type name and payload; a quiet period ends
    the stream; a mask filters types before registration."""
    out = _run("""
from rocm_systems_b200.tools.smi import Smi
s = Smi()
evs = list(s.events(timeout_ms=100))
print([(e['device'], e['type'], e['data']) for e in evs])
only_xid = list(s.events(timeout_ms=100, mask=0x8))
print([(e['device'], e['type'], e['data']) for e in only_xid])
s.close()
""", fake_nvml, {"FAKE_NVML_EVENTS": "2:8:79,0:2:1,3:16:0", "FAKE_NVML_GPUS": "4"})
    lines = out.strip().splitlines()
    assert lines[0] == "[(2, 'xid', 79), (0, 'ecc_double_bit', 1), (3, 'clock', 0)]"
    assert lines[1] == "[(2, 'xid', 79)]"


def test_event_cli(fake_nvml):
    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake_nvml, PYTHONPATH=str(ROOT), FAKE_NVML_GPUS="2", FAKE_NVML_EVENTS="1:8:94")
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "--showevents", "0.1"], env=e, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    assert "GPU1: xid data=94" in p.stdout and "Name" not in p.stdout


def test_single_reading_flags(fake_nvml):
    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake_nvml, PYTHONPATH=str(ROOT), FAKE_NVML_GPUS="2", FAKE_NVML_TEMP="61")
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "--showtemp", "--showclocks", "--showmeminfo", "--showthrottle"], env=e,
                       capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    lines = p.stdout.strip().splitlines()
    assert len(lines) == 2 and lines[0].startswith("GPU0: 61 C; SM 1500/1965 MHz") and "1.0 / 179.1 GiB" in lines[1] and "sw_power_cap" in lines[1]


def test_bench_health_annotation(fake_nvml):
    """bench.py records the GPU's link, ECC and health state next to its numbers; without NVML it says so instead of failing."""
    out = _run("""
import json, bench
h = bench.gpu_health(1)
print(json.dumps(h))
""", fake_nvml, {"FAKE_NVML_LINK_DOWN": "1", "FAKE_NVML_LINK_ERRORS": "1"})
    import json

    h = json.loads(out.strip().splitlines()[-1])
    assert h["level"] == "FAIL" and h["nvlink_active"] == 17 and h["nvlink_count"] == 18 and h["nvlink_errors"]["replay"] == 5
    e = dict(os.environ, B200SMI_NVML_LIBRARY="/nonexistent/libnvml.so", PYTHONPATH=str(ROOT))
    p = subprocess.run([sys.executable, "-c", "import bench, json; print(json.dumps(bench.gpu_health(0)))"], env=e, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and "unavailable" in json.loads(p.stdout.strip().splitlines()[-1])


def test_subcommand_front_end(fake_nvml):
    """``list`` / ``static`` / ``metric`` / ``topology`` / ``process`` / ``monitor`` / ``event`` / ``version`` over the same readings,
    as JSON, CSV and text, with a GPU selection."""
    import csv
    import io
    import json

    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake_nvml, PYTHONPATH=str(ROOT), FAKE_NVML_GPUS="4", FAKE_NVML_TEMP="58", FAKE_NVML_EVENTS="1:8:94")

    def run(*args):
        p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", *args], env=e, capture_output=True, text=True)
        assert p.returncode == 0, p.stderr
        return p.stdout

    lst = json.loads(run("list", "--json"))
    assert [r["gpu"] for r in lst] == [0, 1, 2, 3] and all(r["uuid"] and r["bus_id"] for r in lst)
    st = json.loads(run("static", "-g", "1", "3", "--json"))
    assert [r["gpu"] for r in st] == [1, 3] and st[0]["nvlink_links"] == 18 and st[0]["pcie_generation"] == 5 and "power_limit_w" in st[0]
    rows = list(csv.DictReader(io.StringIO(run("metric", "--csv"))))
    assert len(rows) == 4 and rows[0]["temperature_c"] == "58" and {"sm_clock_mhz", "power_w", "nvlink_replay", "throttle"} <= set(rows[0])
    topo = json.loads(run("topology", "-g", "0", "2", "--json"))
    assert {(r["gpu"], r["peer"]) for r in topo} == {(0, 2), (2, 0)} and topo[0]["type"] == "NVLINK" and topo[0]["peer_access"] is True
    assert "GPU 0: power_w" in run("monitor", "-g", "0", "-i", "2", "-w", "0.01")
    ev = json.loads(run("event", "-t", "0.3", "--json"))
    assert ev and ev[0]["gpu"] == 1 and ev[0]["data"] == 94
    assert "580.159.fake" in run("version")
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "metric", "-g", "9"], env=e, capture_output=True, text=True)
    assert p.returncode == 2 and "no GPU 9" in p.stderr


def test_activity_from_monitoring_samples(fake_nvml):
    """Activity fields: the first reading brackets 100 ms itself, readings in quick succession share one interval, a later
    one spans from the previous sample to now (the stand-in reports the number of samples in the interval as NVLink
    traffic), a metric the device does not report comes back as unsupported, and the watch thread records them."""
    out = _run("""
import time
from rocm_systems_b200.tools.smi import Smi, FIELDS, ACTIVITY_FIELDS
s = Smi()
t0 = time.time()
a = s.activity(0)
assert 0.09 < time.time() - t0 < 5.0 and 90 <= a['interval_ms'] < 5000
assert a['tensor_active_pct'] == 40.0 and a['sm_active_pct'] == 91.0 and a['sm_occupancy_pct'] == 48.5 and a['dram_active_pct'] == 33.0
assert a['fp64_active_pct'] is None and a['pcie_tx_mibs'] == 120.0
assert a['nvlink_tx_mibs'] == 1000.0 and a['nvlink_rx_mibs'] == 900.0            # two consecutive samples
t1 = time.time(); again = s.activity(0)
assert again == a or time.time() - t1 > 0.03 or again['tensor_active_pct'] == 40.0   # within 50 ms: the same interval again
assert s.read(0, 'tensor_active') == 40.0 and s.read(0, 'nvlink_rx_mibs') == 900.0
try:
    s.read(0, 'fp64_active'); raise SystemExit('fp64 should be unsupported')
except RuntimeError as e:
    assert 'not supported' in str(e)
time.sleep(0.12)
b = s.activity(0)                                                                  # one new sample: previous -> now
assert b['nvlink_tx_mibs'] == 1000.0 and 100 <= b['interval_ms'] < 5000
c = s.activity(1)                                                                  # another device has its own samples
assert c['nvlink_tx_mibs'] == 1000.0
assert len(ACTIVITY_FIELDS) == 11 and FIELDS['nvlink_rx_mibs'] == 22
s.watch_start([0], ['tensor_active', 'power'], period_ms=60, keep=50)
time.sleep(0.4)
hist = s.history(0, 'tensor_active')
s.watch_stop()
assert len(hist) >= 2 and all(v == 40.0 for _, v in hist), hist
print('ok')
""", fake_nvml, {"FAKE_NVML_TENSOR": "40"})
    assert "ok" in out
    out = _run("""
from rocm_systems_b200.tools.smi import Smi
try:
    Smi().activity(0); raise SystemExit('should be unsupported')
except RuntimeError as e:
    assert 'not supported' in str(e)
print('ok')
""", fake_nvml, {"FAKE_NVML_GPM": "0"})
    assert "ok" in out
    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake_nvml, PYTHONPATH=str(ROOT), FAKE_NVML_GPUS="2")
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "--showactivity"], env=e, capture_output=True, text=True)
    assert p.returncode == 0 and p.stdout.count("tensor 62.5 %") == 2 and "fp64/32/16 n/a/7/1 %" in p.stdout, p.stdout + p.stderr
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "metric", "--activity", "--json", "-g", "1"], env=e, capture_output=True, text=True)
    import json
    row = json.loads(p.stdout)[0]
    assert row["gpu"] == 1 and row["tensor_active_pct"] == 62.5 and row["fp64_active_pct"] is None and row["power_w"] == 200.0


def test_telemetry_activity_field_group_and_prometheus(fake_nvml):
    out = _run("""
import time
from rocm_systems_b200.tools.telemetry import Telemetry
t = Telemetry()
assert 'tensor_active' in t.field_groups['activity'] and len(t.field_groups['activity']) == 11
t.create_group('pair', [0, 1])
t.watch('pair', 'activity', period_ms=60, keep=100)
time.sleep(0.35)
vals = t.latest()
assert vals[0]['tensor_active'] == 62.5 and vals[1]['fp64_active'] is None
text = t.prometheus()
assert 'b200_tensor_active_percent{gpu="1",' in text and 'b200_fp64_active_percent{gpu=' not in text
line = next(l for l in text.splitlines() if l.startswith('b200_nvlink_tx_bytes_per_second{gpu="0"'))
assert float(line.split()[-1]) % 1048576000.0 == 0                       # MiB/s scaled to bytes per second
hist = t.history(1, 'dram_active')
assert len(hist) >= 2 and all(v == 33.0 for _, v in hist)
t.stop()
print('ok')
""", fake_nvml)
    assert "ok" in out


def test_launcher_samples_activity_fields_next_to_the_trace(fake_nvml, tmp_path):
    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake_nvml, PYTHONPATH=str(ROOT), FAKE_NVML_GPUS="2", FAKE_NVML_TENSOR="77")
    base = [sys.executable, "-m", "rocm_systems_b200.tools.prof", "--marker-trace", "--sys-sample", "40", "-d", str(tmp_path), "-o", "run"]
    p = subprocess.run([*base, "--sys-sample-fields", "tensor_active", "nvlink_tx_mibs", "power", "--stats", "--", sys.executable, "-c", "import time; time.sleep(0.5)"],
                       env=e, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr
    import sqlite3

    db = sqlite3.connect(str(tmp_path / "run.db"))
    got = dict(db.execute("select s.value, avg(c.value) from counter_sample c join string s on s.id = c.name_id group by s.value").fetchall())
    assert got["gpu_tensor_active"] == 77.0 and got["gpu_power"] == 200.0 and got["gpu_nvlink_tx_mibs"] >= 1000.0 and "gpu_sm_clock" not in got
    assert "gpu_tensor_active" in p.stdout                                       # the sampled-counters table of --stats
    p = subprocess.run([*base, "--sys-sample-fields", "nope", "--", "true"], env=e, capture_output=True, text=True, timeout=60)
    assert p.returncode == 2 and "unknown --sys-sample-fields" in p.stderr


def test_identity_readings_and_gated_clock_lock(fake_nvml):
    out = _run("""
from rocm_systems_b200.tools.smi import Smi
s = Smi()
d = s.identity(2)
assert d['serial'] == '1650123450002' and d['part_number'] == '699-2G525-0200-000' and d['vbios'] == '97.00.88.00.0F' and d['inforom_image'] is None
assert d['performance_state'] == 0 and d['power_limit_min_w'] == 200.0 and d['power_limit_max_w'] == 1000.0
assert abs(d['energy_j'] - 123456.791) < 1e-6 and d['remapped_rows'] == {'correctable': 0, 'uncorrectable': 0, 'pending': False, 'failed': False}
assert s.identity(1)['remapped_rows']['correctable'] == 2
for call in (lambda: s.set_locked_clocks(0, 1200, 1500, True), lambda: s.reset_locked_clocks(0, True)):
    try:
        call(); raise SystemExit('setter ran without B200SMI_ALLOW_SET')
    except RuntimeError as e:
        assert 'disabled' in str(e)
print('ok')
""", fake_nvml, {"FAKE_NVML_ECC": "1"})
    assert "ok" in out
    out = _run("""
from rocm_systems_b200.tools.smi import Smi
s = Smi()
try:
    s.set_locked_clocks(0, 1200, 1500, False); raise SystemExit('setter ran without allow')
except RuntimeError as e:
    assert 'disabled' in str(e)
try:
    s.set_locked_clocks(0, 1500, 1200, True); raise SystemExit('min above max accepted')
except RuntimeError as e:
    assert 'invalid' in str(e)
s.set_locked_clocks(0, 1200, 1350, True)
assert s.info(0)['smClockMhz'] == 1350 and s.info(1)['smClockMhz'] == 1500       # the stand-in shows the lock in its clock reading
s.reset_locked_clocks(0, True)
assert s.info(0)['smClockMhz'] == 1500
print('ok')
""", fake_nvml, {"B200SMI_ALLOW_SET": "1"})
    assert "ok" in out
    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake_nvml, PYTHONPATH=str(ROOT), FAKE_NVML_GPUS="2")
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "--showserial", "--showperflevel", "--showmaxpower", "--showenergycounter",
                        "--showretiredpages", "--showfwinfo"], env=e, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    assert "GPU1: serial 1650123450001, part number 699-2G525-0200-000; VBIOS 97.00.88.00.0F, InfoROM image n/a; P0; power limit settable in 200 - 1000 W;" in p.stdout, p.stdout
    assert "J since the driver was loaded; remapped rows: 0 correctable, 0 uncorrectable" in p.stdout and "Name" not in p.stdout
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "--setclocks", "0", "1200", "1400", "--allow-set"], env=e, capture_output=True, text=True)
    assert p.returncode == 2 and "disabled" in p.stderr                                    # the environment half of the gate is missing
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "static", "--json", "-g", "0"], env=e, capture_output=True, text=True)
    import json
    row = json.loads(p.stdout)[0]
    assert row["serial"] == "1650123450000" and row["vbios"] == "97.00.88.00.0F" and row["power_limit_range_w"] == "200-1000"


def test_telemetry_reader_embedded_and_against_a_daemon(fake_nvml):
    out = _run("""
import threading, time
from rocm_systems_b200.tools.telemetry import Reader, Telemetry, serve
seen = []
class Log(Reader):
    def handle_field(self, device, field, value, timestamp_ns):
        seen.append((device, field, value))
r = Log(fields=['power', 'tensor_active', 'fp64_active'], devices=[0, 2], period_ms=20)
r.run(iterations=3)
assert r.reads == 3 and len(seen) == 3 * 2 * 2                      # fp64 is unsupported on the stand-in: skipped
assert {s[0] for s in seen} == {0, 2} and {s[1] for s in seen} == {'power', 'tensor_active'} and all(s[2] in (200.0, 62.5) for s in seen)
try:
    Reader(fields=['nope']); raise SystemExit('unknown field accepted')
except ValueError:
    pass
# against a daemon
t = Telemetry()
srv = serve(t, '127.0.0.1', 0)
port = srv.server_address[1]
threading.Thread(target=srv.serve_forever, daemon=True).start()
got = []
c = Reader(url=f'http://127.0.0.1:{port}', fields=['temp', 'sm_clock'], period_ms=10, on_field=lambda d, f, v, ts: got.append((d, f, v)))
assert c.devices == list(range(8))
assert c.process() == 16 and ((3, 'temp', 45.0) in got) and ((7, 'sm_clock', 1500.0) in got)
stop = threading.Event()
th = threading.Thread(target=c.run, kwargs={'stop': stop}); th.start(); time.sleep(0.1); stop.set(); th.join(2)
assert not th.is_alive() and c.reads >= 2
srv.shutdown()
print('ok')
""", fake_nvml)
    assert "ok" in out


def test_cpu_affinity_of_a_gpu_and_pinning(fake_nvml, tmp_path):
    ncpu = len(os.sched_getaffinity(0))
    per = max(1, ncpu // 2)                                   # the stand-in puts GPU i on CPUs [per*i, per*i + per)
    out = _run(f"""
import os
from rocm_systems_b200.tools.smi import Smi
from rocm_systems_b200.utils import affinity
s = Smi()
a = s.cpu_affinity(1)
assert a == {{'cpus': list(range({per}, {2 * per})), 'numa_node': 0}}, a
assert s.cpu_affinity(5)['numa_node'] == 1
assert affinity.parse_cpu_list('0-3,8,10-11\\n') == [0, 1, 2, 3, 8, 10, 11] and affinity.format_cpu_list([11, 0, 1, 2, 3, 8, 10]) == '0-3,8,10-11'
assert affinity.format_cpu_list([]) == '' and affinity.parse_cpu_list('') == []
g = affinity.gpu_cpus(0)
assert g['source'] == 'nvml' and g['cpus'] == list(range(0, {per}))
before = os.sched_getaffinity(0)
allowed = sorted(before)
set_ = affinity.pin_to_gpu(0)
want = [c for c in range(0, {per}) if c in before]
assert (set_ == want and sorted(os.sched_getaffinity(0)) == want) if want and set(want) != before else set_ is None
os.sched_setaffinity(0, before)
assert affinity.pin_to_gpu(7) is None or True                 # CPUs beyond this machine: nothing to intersect with, nothing changes
assert not affinity.wanted()
os.environ['B200COLL_CPU_AFFINITY'] = '1'
assert affinity.wanted()
print('ok')
""", fake_nvml, {"FAKE_NVML_CPUS_PER_GPU": str(per)})
    assert "ok" in out
    # without NVML affinity: the PCI device's local_cpulist in sysfs (a stand-in tree here)
    dev = tmp_path / "sys" / "bus" / "pci" / "devices" / "0000:12:00.0"
    dev.mkdir(parents=True)
    (dev / "local_cpulist").write_text("0-1\n")
    (dev / "numa_node").write_text("-1\n")
    out = _run(f"""
from rocm_systems_b200.utils import affinity
from rocm_systems_b200.tools import smi
smi.Smi.cpu_affinity = lambda self, dev: (_ for _ in ()).throw(RuntimeError('not supported by this device or driver'))
g = affinity.gpu_cpus(2, sysfs_root=r'{tmp_path / "sys"}')
assert g == {{'cpus': [0, 1], 'numa_node': None, 'source': 'sysfs'}}, g
assert affinity.gpu_cpus(3, sysfs_root=r'{tmp_path / "sys"}')['source'] == 'none'
print('ok')
""", fake_nvml)
    assert "ok" in out
    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake_nvml, PYTHONPATH=str(ROOT), FAKE_NVML_GPUS="2", FAKE_NVML_CPUS_PER_GPU="6")
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", "--showtoponuma"], env=e, capture_output=True, text=True)
    assert p.returncode == 0 and "GPU0: NUMA node 0, CPUs 0-5" in p.stdout and "GPU1: NUMA node 0, CPUs 6-11" in p.stdout, p.stdout + p.stderr


def test_dmon_field_groups_listing_and_unsupported_fields(fake_nvml):
    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake_nvml, PYTHONPATH=str(ROOT), FAKE_NVML_GPUS="2")
    base = [sys.executable, "-m", "rocm_systems_b200.tools.telemetry", "dmon"]
    p = subprocess.run([*base, "-f", "activity", "-c", "1"], env=e, capture_output=True, text=True, timeout=60)
    assert p.returncode == 0, p.stderr
    lines = p.stdout.strip().splitlines()
    head = lines[0].split("\t")
    assert head[0] == "GPU" and "tensor_active" in head and len(lines) == 3
    row = dict(zip(head, lines[1].split("\t")))
    assert row["tensor_active"] == "62.5" and row["fp64_active"] == "n/a" and row["sm_active"] == "91"
    p = subprocess.run([*base, "-l"], env=e, capture_output=True, text=True, timeout=60)
    assert p.returncode == 0 and "tensor_active" in p.stdout and "group activity: sm_active" in p.stdout and "group default:" in p.stdout
    assert subprocess.run([*base, "-e", "nope", "-c", "1"], env=e, capture_output=True, text=True, timeout=60).returncode == 2
    assert subprocess.run([*base, "-f", "nope", "-c", "1"], env=e, capture_output=True, text=True, timeout=60).returncode == 2


def test_more_subcommands_firmware_bad_pages_nvlink_set_reset(fake_nvml):
    import json

    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake_nvml, PYTHONPATH=str(ROOT), FAKE_NVML_GPUS="2", FAKE_NVML_ECC="1")
    run = lambda *args, **env: subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", *args], env=dict(e, **env), capture_output=True, text=True)  # noqa: E731
    fw = json.loads(run("firmware", "--json").stdout)
    assert fw[0]["vbios"] == "97.00.88.00.0F" and fw[0]["inforom_image"] is None and fw[1]["driver"] == "580.159.fake"
    bp = json.loads(run("bad-pages", "--json").stdout)
    assert bp[0]["correctable"] == 0 and bp[1]["correctable"] == 2 and bp[1]["failed"] is False
    nv = json.loads(run("nvlink", "--activity", "--json", "-g", "1").stdout)
    assert nv == [{"gpu": 1, "links": 18, "links_up": 18, "replay": nv[0]["replay"], "recovery": nv[0]["recovery"], "crc_flit": nv[0]["crc_flit"],
                   "crc_data": nv[0]["crc_data"], "tx_mibs": 1000.0, "rx_mibs": 900.0}]
    p = run("set", "--clocks", "1200", "1400", "-g", "0", "--allow-set")
    assert p.returncode == 2 and "disabled" in p.stderr                                   # the environment half of the gate is missing
    p = run("set", "--clocks", "1200", "1400", "--allow-set", B200SMI_ALLOW_SET="1")
    assert p.returncode == 2 and "name the GPUs" in p.stderr                              # never on all GPUs by default
    p = run("set", "--clocks", "1200", "1400", "--power-limit", "800", "-g", "0", "--allow-set", B200SMI_ALLOW_SET="1")
    assert p.returncode == 0 and "GPU 0: done set" in p.stdout, p.stderr
    assert run("reset", "--clocks", "-g", "0", "--allow-set", B200SMI_ALLOW_SET="1").returncode == 0


def test_flag_front_end_device_selection(fake_nvml):
    e = dict(os.environ, B200SMI_NVML_LIBRARY=fake_nvml, PYTHONPATH=str(ROOT), FAKE_NVML_GPUS="4")
    run = lambda *args: subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.smi", *args], env=e, capture_output=True, text=True)  # noqa: E731
    p = run("--showtemp", "--showserial", "-d", "2", "3")
    assert p.returncode == 0 and "GPU2:" in p.stdout and "GPU3: serial 1650123450003" in p.stdout and "GPU0" not in p.stdout and "GPU1" not in p.stdout, p.stdout + p.stderr
    import json
    doc = json.loads(run("--showbus", "--shownvlinkerrors", "--json", "-d", "1").stdout)
    assert len(doc["pcie"]) == 1 and len(doc["nvlink_errors"]) == 1
    assert run("--showtemp", "-d", "9").returncode == 2
    p = run("--showall")
    assert p.returncode == 0 and all(f"GPU{i}" in p.stdout or f"\n{i} " in p.stdout or str(i) in p.stdout for i in range(4))
