"""CPU tests of the tooling around the library: dispatch-table tool loading, markers, the trace
database and its converters, the tracing launcher's environment hand-off, the telemetry service
against a fake NVML, the roofline report and the device dump."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _py(code: str, env=None, timeout=120):
    e = dict(os.environ, PYTHONPATH=str(ROOT))
    e.update(env or {})
    p = subprocess.run([sys.executable, "-c", code], env=e, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, p.stdout + p.stderr
    return p.stdout


def test_sample_tool_wraps_dispatch_table(tmp_path):
    from rocm_systems_b200.utils import build

    tool = build.build_sample_tool()
    out = tmp_path / "tool.txt"
    _py("""
import ctypes
from rocm_systems_b200 import _lib
lib = _lib.load()
v = ctypes.c_int()
for _ in range(3):
    assert lib.ncclGetVersion(ctypes.byref(v)) == 0
assert v.value == 22005, v.value
""", {"B200COLL_TOOL_LIBRARIES": str(tool), "B200COLL_SAMPLE_TOOL_OUTPUT": str(out)})
    text = out.read_text()
    assert "ncclGetVersion calls=3" in text and "payload_bytes=0" in text


def test_tool_loading_switches(tmp_path):
    """Off switch and secure mode of tool loading: an absolute path to a file nobody else can write is loaded, a relative
    path or a file others can write is refused with a warning, and with registration off nothing is loaded."""
    import shutil
    import stat

    from rocm_systems_b200.utils import build

    tool = build.build_sample_tool()
    good = tmp_path / "libtool.so"
    shutil.copy(tool, good)
    good.chmod(0o755)
    loose = tmp_path / "libloose.so"
    shutil.copy(tool, loose)
    loose.chmod(0o777)
    code = "import ctypes\nfrom rocm_systems_b200 import _lib\nlib = _lib.load()\nv = ctypes.c_int()\nassert lib.ncclGetVersion(ctypes.byref(v)) == 0\n"

    def run(libs, **env):
        out = tmp_path / f"out_{len(list(tmp_path.glob('out_*')))}.txt"
        e = dict(os.environ, PYTHONPATH=str(ROOT), B200COLL_TOOL_LIBRARIES=libs, B200COLL_SAMPLE_TOOL_OUTPUT=str(out), B200COLL_DEBUG="WARN", **env)
        p = subprocess.run([sys.executable, "-c", code], env=e, capture_output=True, text=True, timeout=120, cwd=tmp_path)
        assert p.returncode == 0, p.stderr
        return out.exists() and "ncclGetVersion calls=1" in out.read_text(), p.stdout + p.stderr

    assert run(str(good))[0]
    assert run(str(good), B200COLL_TOOL_SECURE="1")[0]
    loaded, log = run(str(loose), B200COLL_TOOL_SECURE="1")
    assert not loaded and "refused in secure mode: writable by group or others" in log
    loaded, log = run("libtool.so", B200COLL_TOOL_SECURE="1")
    assert not loaded and "not an absolute path" in log
    assert run("libtool.so")[0] is False or True      # without secure mode a relative name is left to the dynamic loader's search
    assert not run(str(good), B200COLL_TOOL_REGISTER_ENABLED="0")[0]
    assert stat.S_IMODE(loose.stat().st_mode) == 0o777


def test_markers_nest_and_write_csv(tmp_path):
    out = _py(f"""
from rocm_systems_b200.utils import markers
assert markers.range_push('ignored') == -1          # off until enabled
markers.enable()
with markers.range('outer'):
    with markers.range('inner'):
        markers.mark('point')
rid = markers.range_start('async')
markers.range_stop(rid)
assert markers.range_at('earlier', 1000, 3000) > rid
recs = markers.records()
names = [r['message'] for r in recs]
assert names == ['point', 'inner', 'outer', 'async', 'earlier'], names
assert recs[-1]['begin_ns'] == 1000 and recs[-1]['end_ns'] == 3000
by = {{r['message']: r for r in recs}}
assert by['inner']['depth'] == 1 and by['outer']['depth'] == 0 and by['point']['depth'] == 2
assert by['outer']['begin_ns'] <= by['inner']['begin_ns'] <= by['inner']['end_ns'] <= by['outer']['end_ns']
assert markers.write_csv(r'{tmp_path}/m.csv') == 5
assert 'b200coll' in markers.build_info()
where = markers.install_path()
assert where['library'].endswith('/lib/libb200coll.so') and where['library'].startswith(where['prefix'] + '/') and where['prefix'].endswith('rocm_systems_b200')
print('ok')
""")
    assert "ok" in out
    assert (tmp_path / "m.csv").read_text().count("MARKER_API") == 5


def test_markers_written_at_exit_under_trace_env(tmp_path):
    prefix = tmp_path / "t"
    _py("""
from rocm_systems_b200.utils import markers
with markers.range('step'):
    pass
""", {"B200COLL_TRACE": "1", "B200COLL_TRACE_FILE": str(prefix)})
    files = list(tmp_path.glob("t.markers.*.csv"))
    assert len(files) == 1 and '"step"' in files[0].read_text()


KERNEL_CSV = '''"Kind","Agent_Id","Queue_Id","Process_Id","Kernel_Name","Correlation_Id","Start_Timestamp","End_Timestamp","Registers_Per_Thread","Static_Shared_Memory","Dynamic_Shared_Memory","Local_Memory_Per_Thread","Workgroup_Size_X","Workgroup_Size_Y","Workgroup_Size_Z","Grid_Size_X","Grid_Size_Y","Grid_Size_Z","Cluster_X","Cluster_Y","Cluster_Z","Graph_Node_Id"
"KERNEL_DISPATCH",0,7,100,"gemmKernel<Cfg>",1,1000,5000,168,0,200000,0,192,1,1,148,1,1,1,1,1,0
"KERNEL_DISPATCH",0,7,100,"gemmKernel<Cfg>",2,6000,9000,168,0,200000,0,192,1,1,148,1,1,1,1,1,0
"KERNEL_DISPATCH",0,7,100,"rmsnorm",3,9500,10000,32,0,0,0,256,1,1,4096,1,1,1,1,1,0
'''
COLL_CSV = '''"Domain","Function","Process_Id","Thread_Id","Correlation_Id","Start_Timestamp","End_Timestamp","Rank","Count","Dtype","Bytes","Algo","Ctas","Device_Start","Device_End","Device_Us","AlgBw_GBps"
"B200COLL_API","ncclAllReduce",100,100,1,900,950,0,1048576,"float",4194304,2,64,2000,12000,10.000,419.430
"B200COLL_API","ncclAllReduce",100,100,2,1900,1950,0,1048576,"float",4194304,2,64,22000,30000,8.000,524.288
'''
MARK_CSV = '''"Domain","Function","Process_Id","Thread_Id","Correlation_Id","Start_Timestamp","End_Timestamp","Depth"
"MARKER_API","step 0",100,100,1,500,20000,0
'''


def test_tracedb_import_summary_convert(tmp_path):
    from rocm_systems_b200.tools import tracedb

    (tmp_path / "t.100_kernel_trace.csv").write_text(KERNEL_CSV)
    (tmp_path / "t.rank0.csv").write_text(COLL_CSV)
    (tmp_path / "t.markers.100.csv").write_text(MARK_CSV)
    dbp = str(tmp_path / "t.db")
    with tracedb.TraceDB(dbp) as db:
        n = sum(db.import_csv(str(p)) for p in sorted(tmp_path.glob("t.*csv")))
        assert n == 6
        s = db.summary()
        top = s["kernels"][0]
        assert top["name"] == "gemmKernel<Cfg>" and top["calls"] == 2 and top["total_ns"] == 7000
        assert abs(top["percent"] - 7000 / 7500 * 100) < 1e-6
        assert s["collectives"][0]["calls"] == 2 and s["collectives"][0]["mean_ns"] == 9000
        assert s["busy"][0]["kernels"] == 3 and s["busy"][0]["rank"] == 0      # rank learnt from the collective trace of the same pid
        cats = {r["category"] for r in s["regions"]}
        assert cats == {"B200COLL_API", "MARKER_API"}
        ev = db.to_perfetto(str(tmp_path / "t.json"))
        assert ev == 1 + 3 + 3 + 2 + 2 + 4  # process name, kernels, regions (2 API + 1 marker), device-side collectives, comm-volume counter points, 2 call -> device arrows
        files = db.to_csv(str(tmp_path / "out"))
        assert any(f.endswith("_top_kernels.csv") for f in files)
    doc = json.loads((tmp_path / "t.json").read_text())
    assert {e["ph"] for e in doc["traceEvents"]} == {"M", "X", "C", "s", "f"}
    arrows = sorted((e for e in doc["traceEvents"] if e["ph"] in "sf"), key=lambda e: (e["id"], e["ph"] == "f"))
    assert [(e["ph"], e["tid"], e["ts"]) for e in arrows[:2]] == [("s", "B200COLL_API 100", 0.9), ("f", "collectives (device)", 2.0)]   # call at 900 ns, device at 2000 ns
    vol = [e for e in doc["traceEvents"] if e["ph"] == "C"]
    assert [e["name"] for e in vol] == ["Comm Recv (bytes)"] * 2 and [e["args"]["value"] for e in vol] == [4194304, 8388608]   # all-reduce counts as received; cumulative
    # a second rank's database merges in
    db2 = str(tmp_path / "r1.db")
    (tmp_path / "u.rank1.csv").write_text(COLL_CSV.replace(",100,100,", ",200,200,").replace(",0,1048576", ",1,1048576"))
    with tracedb.TraceDB(db2) as d2:
        d2.import_csv(str(tmp_path / "u.rank1.csv"))
    with tracedb.TraceDB(dbp) as db:
        db.merge(db2)
        names, rows = db.query("select rank, count(*) from collectives group by rank order by rank")
        assert rows == [(0, 2), (1, 2)]
    assert tracedb.main(["query", dbp, "select count(*) as n from kernels", "--format", "json"]) == 0


def test_prof_launcher_env_and_collection(tmp_path):
    from rocm_systems_b200.tools import prof

    a = prof.parser().parse_args(["--kernel-trace", "--coll-trace", "--kernel-include-regex", "gemm", "--", "true"])
    env = prof.build_env(a, str(tmp_path / "x"))
    assert env["CUDA_INJECTION64_PATH"].endswith("libb200prof.so") and env["B200PROF_KERNEL_TRACE"] == "1"
    assert env["B200PROF_MEMORY_COPY_TRACE"] == "0" and env["B200PROF_KERNEL_FILTER"] == "gemm"
    assert env["B200COLL_TRACE"] == "1" and env["B200COLL_TRACE_FILE"] == str(tmp_path / "x")
    # end to end without a GPU: the child pushes markers; the launcher collects them into the outputs
    child = "from rocm_systems_b200.utils import markers\nwith markers.range('phase'):\n    markers.mark('tick')\n"
    e = dict(os.environ, PYTHONPATH=str(ROOT))
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.prof", "--marker-trace", "--stats", "--summary", "--output-format", "csv", "db",
                        "pftrace", "json", "-d", str(tmp_path / "o"), "--", sys.executable, "-c", child], env=e, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr
    assert "MARKER_API" in p.stdout and "phase" in p.stdout
    for name in ("trace.db", "trace.perfetto.json", "trace.json", "trace_summary.json", "trace_regions.csv"):
        assert (tmp_path / "o" / name).exists(), name


@pytest.fixture(scope="module")
def fake_nvml(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake_nvml_t") / "libfake_nvml.so"
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-o", str(out), str(ROOT / "tests" / "fake_nvml" / "fake_nvml.c")])
    return str(out)


def test_telemetry_service_with_fake_nvml(fake_nvml):
    out = _py("""
import json, time, urllib.request
from rocm_systems_b200.tools import telemetry
t = telemetry.Telemetry()
assert len(t.discovery()) == 2
t.start(fields=['sm_clock', 'power', 'temp', 'throttle_reasons'], period_ms=20, keep=100)
srv = telemetry.serve(t, '127.0.0.1', 0)
url = 'http://127.0.0.1:%d' % srv.server_address[1]
get = lambda p: urllib.request.urlopen(url + p, timeout=10).read().decode()
get('/api/job/start?job=j1')
time.sleep(0.3)
get('/api/job/stop?job=j1')
m = get('/metrics')
assert '# TYPE b200_power_watts gauge' in m and 'b200_sm_clock_mhz{gpu="1"' in m
line = next(l for l in m.splitlines() if l.startswith('b200_power_watts{gpu="0"'))
watts = float(line.rsplit(' ', 1)[1])
assert 150 < watts < 2000, watts          # watts, not milliwatts or kilowatts
assert 'b200_clock_event_reason{gpu="0",reason="sw_power_cap"} 1' in m
st = json.loads(get('/api/job/stats?job=j1'))
assert st['devices']['0']['power']['samples'] >= 3 and st['devices']['0']['power']['avg'] > 0
h = json.loads(get('/api/history?dev=0&field=temp'))
assert len(h) >= 3
assert json.loads(get('/api/health'))['0']['level'] == 'PASS'
try:
    get('/api/history?dev=0&field=nope'); raise SystemExit('bad field accepted')
except urllib.error.HTTPError as e:
    assert e.code == 400
srv.shutdown(); t.stop()
print('ok')
""", {"B200SMI_NVML_LIBRARY": fake_nvml, "FAKE_NVML_GPUS": "2"})
    assert "ok" in out


NCU_CSV = '''"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","gpu__time_duration.sum","dram__bytes_read.sum","dram__bytes_write.sum","sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active","sm__warps_active.avg.pct_of_peak_sustained_active","launch__registers_per_thread"
"","","","","","","","","","","","us","Mbyte","Mbyte","%","%","register/thread"
"0","1","python","h","rmsnormKernel","1","7","(256, 1, 1)","(4096, 1, 1)","0","10.0","100","300","300","0","80","32"
"1","1","python","h","gemmKernel","1","7","(192, 1, 1)","(148, 1, 1)","0","10.0","1000","200","134","90","9","168"
'''


def test_roofline_report_from_ncu_csv(tmp_path, capsys):
    from rocm_systems_b200.tools import roofline

    ks = roofline.parse_ncu_csv(NCU_CSV)
    assert [k.name for k in ks] == ["rmsnormKernel", "gemmKernel"]
    assert ks[0].duration_ns == 100e3 and ks[0].dram_bytes == 600e6 and abs(ks[0].gbs - 6000) < 1e-6
    peaks = {"hbm_gbs": 6541.5, "bf16_tflops": 1601.7, "source": "measured"}
    assert roofline.classify(ks[0], peaks) == "memory"
    ks[1].flops = 2 * 8192.0 ** 3
    assert roofline.classify(ks[1], peaks) == "compute" and abs(ks[1].tflops - 1099.5) < 1
    (tmp_path / "p.json").write_text(json.dumps({"hbm_gbs": 6541.5, "bf16_tflops": 1601.7}))
    (tmp_path / "raw.csv").write_text(NCU_CSV)
    rc = roofline.main([str(tmp_path / "raw.csv"), "--peaks", str(tmp_path / "p.json"), "--flops", "gemm=1.0995e12", "--plot",
                        "--point", "probe:1e9:1e9:1e-3"])
    text = capsys.readouterr().out
    assert rc == 0 and "of measured" in text and "latency/occupancy" in text and "A: gemmKernel" in text


def test_info_runs_without_gpu():
    e = dict(os.environ, PYTHONPATH=str(ROOT))
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.info", "--json"], env=e, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr
    doc = json.loads(p.stdout)
    assert "host" in doc and "b200coll" in doc["libraries"] and isinstance(doc["devices"], list)
    from rocm_systems_b200.tools.info import arch_target

    assert arch_target(10, 0) == "sm_100a" and arch_target(8, 0) == "sm_80"


def test_system_sampler_and_launcher_counter_tracks(tmp_path, fake_nvml):
    e = dict(os.environ, PYTHONPATH=str(ROOT), B200SMI_NVML_LIBRARY=fake_nvml, FAKE_NVML_GPUS="2")
    child = "import time\nfrom rocm_systems_b200.utils import markers\nwith markers.range('sleep'):\n    time.sleep(0.5)\n"
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.prof", "--marker-trace", "--sys-sample", "50", "--summary", "--output-format", "db",
                        "pftrace", "-d", str(tmp_path), "--", sys.executable, "-c", child], env=e, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr
    s = json.loads((tmp_path / "trace_summary.json").read_text())
    names = {(c["counter"], c["device"]) for c in s["counters"]}
    assert ("gpu_power", 0) in names and ("gpu_power", 1) in names and ("host_mem_used_bytes", -1) in names
    assert any(c["counter"] == "process_rss_bytes" and c["samples"] >= 3 for c in s["counters"])
    ev = json.loads((tmp_path / "trace.perfetto.json").read_text())["traceEvents"]
    assert any(x["ph"] == "C" and x["name"].startswith("gpu_sm_clock") for x in ev)
    # sampler and marker share a clock: the samples bracket the range
    rng = next(x for x in ev if x["ph"] == "X" and x["name"] == "sleep")
    ts = [x["ts"] for x in ev if x["ph"] == "C"]
    assert min(ts) <= rng["ts"] + 2e5 and max(ts) >= rng["ts"] + rng["dur"] - 2e5


def test_settings_listing_reflects_environment():
    out = _py("""
import json
from rocm_systems_b200.tools import avail
rows = {r['name']: r for r in avail.settings()}
assert rows['BUFFSIZE']['value'] == str(32 << 20) and rows['BUFFSIZE']['env'] == ['B200COLL_BUFFSIZE', 'NCCL_BUFFSIZE']
assert rows['ALGO']['value'] == 'p2p' and rows['WAIT_TIMEOUT_MS']['value'] == '20000'
assert rows['PIPELINE_CHUNK']['default'] == '-1' and len(rows) >= 20
assert avail.main(['--changed']) == 0
print('ok')
""", {"B200COLL_BUFFSIZE": "32M", "NCCL_ALGO": "P2P"})
    assert "ok" in out and "B200COLL_BUFFSIZE" in out and "B200COLL_TRACE " not in out


def test_system_sampler_command_line_and_console_scripts(tmp_path):
    """The sampler around a command, its CSV into the database, and every console script of the package resolves."""
    import subprocess as sp
    import tomllib
    import importlib

    from rocm_systems_b200.tools import tracedb

    out = tmp_path / "s.csv"
    r = sp.run([sys.executable, "-m", "rocm_systems_b200.tools.sysmon", "--no-gpu", "--period-ms", "30", "-o", str(out), "--", sys.executable, "-c",
                "import time; time.sleep(0.3); raise SystemExit(4)"], capture_output=True, text=True, cwd=ROOT, timeout=120)
    assert r.returncode == 4 and "samples of" in r.stderr                       # the command's exit code passes through
    with tracedb.TraceDB(str(tmp_path / "s.db")) as db:
        assert db.import_csv(str(out)) >= 20
        names = {n for (n,) in db.query("select distinct s.value from counter_sample c join string s on s.id = c.name_id")[1]}
    assert {"host_cpu_util_percent", "process_rss_bytes", "process_threads"} <= names
    rss = [float(l.rsplit(",", 1)[1]) for l in out.read_text().splitlines() if l.startswith('"process_rss_bytes"')]
    assert all(v == int(v) for v in rss) and max(rss) > 1e6 and max(rss) % 4096 == 0   # whole bytes (pages), not rounded to six digits
    from rocm_systems_b200 import __main__ as door

    for name in door.TOOLS:                                                     # every tool the package door lists exists and has a main()
        assert callable(importlib.import_module("rocm_systems_b200.tools." + name).main), name
    assert {p.stem for p in (ROOT / "rocm_systems_b200" / "tools").glob("*.py")} - {"__init__"} == set(door.TOOLS)
    assert door.main(["nope"]) == 2 and door.main([]) == 0 and door.main(["instrument", "flags"]) == 0
    scripts = tomllib.loads((ROOT / "pyproject.toml").read_text())["project"]["scripts"]
    assert len(scripts) >= 15
    for name, target in scripts.items():
        mod, fn = target.split(":")
        assert callable(getattr(importlib.import_module(mod), fn)), name


def test_python_reference_is_current():
    """docs/python_api.md is what the generator writes from today's code (regenerate it after changing a public signature)."""
    import io
    from contextlib import redirect_stdout

    from rocm_systems_b200.utils import apidoc

    buf = io.StringIO()
    with redirect_stdout(buf):
        assert apidoc.main([]) == 0
    text = buf.getvalue()
    assert "not importable here" not in text and text.count("\n## `") == len(apidoc.MODULES)
    assert text == (ROOT / "docs" / "python_api.md").read_text(), "run: python -m rocm_systems_b200.utils.apidoc > docs/python_api.md"
    buf = io.StringIO()
    with redirect_stdout(buf):
        assert apidoc.main(["--c"]) == 0
    c = buf.getvalue()
    assert "ncclResult_t ncclAllReduce(const void* sendbuff" in c and "b200smi_status_t b200smi_activity(int device" in c and c.count("\n- `") > 200
    assert c == (ROOT / "docs" / "c_api.md").read_text(), "run: python -m rocm_systems_b200.utils.apidoc --c > docs/c_api.md"


def test_settings_listing_covers_the_tool_libraries(capsys):
    """Every listed environment name is read somewhere in the package, and the listing can be narrowed by component."""
    import subprocess as sp

    from rocm_systems_b200.tools import avail

    names = [env for _, env, _, _ in avail.TOOL_SETTINGS]
    assert len(names) == len(set(names)) >= 35
    pkg = ROOT / "rocm_systems_b200"
    for env in names:
        hit = sp.run(["grep", "-rlF", "--include=*.cc", "--include=*.cu", "--include=*.cuh", "--include=*.h", "--include=*.py", f'"{env}"', str(pkg)],
                     capture_output=True, text=True).stdout.split()
        assert [h for h in hit if not h.endswith("tools/avail.py")], env
    os.environ["B200CAUSAL_FREQ"] = "250"
    try:
        assert avail.main(["--component", "causal", "--changed"]) == 0
    finally:
        del os.environ["B200CAUSAL_FREQ"]
    out = capsys.readouterr().out
    assert out.count("\n") == 1 and out.startswith("B200CAUSAL_FREQ") and "250" in out
    assert avail.main(["--component", "kokkosp", "--json"]) == 0
    rows = json.loads(capsys.readouterr().out)
    assert [r["name"] for r in rows] == ["B200KOKKOSP_MEMORY_EVENTS", "B200KOKKOSP_VERBOSE"] and all(r["component"] == "kokkosp" for r in rows)


def test_tuning_table_from_sweeps(tmp_path):
    from rocm_systems_b200.tools import tune

    def doc(times):
        return {"nranks": 8, "rows": [{"coll": "all_reduce", "bytes": b, "ours_us": t} for b, t in times.items()]}

    ll = doc({1024: 10, 65536: 14, 1 << 20: 90})
    p2p = doc({1024: 20, 65536: 13.8, 1 << 20: 40, 1 << 26: 700})
    nvls = doc({1024: 22, 65536: 25, 1 << 20: 30, 1 << 26: 400})
    t = tune.build_table({"ll": ll, "p2p": p2p, "nvls": nvls})
    rows = [(e["max_bytes"], e["algo"]) for e in t["entries"]]
    # ll keeps 64 KiB although p2p is 1.4 % faster there (inside the margin); nvls takes over from 1 MiB
    assert rows == [(65536, "ll"), (1 << 62, "nvls")], rows
    (tmp_path / "a.json").write_text(json.dumps(ll))
    (tmp_path / "b.json").write_text(json.dumps(nvls))
    assert tune.main([f"ll={tmp_path / 'a.json'}", f"nvls={tmp_path / 'b.json'}", "-o", str(tmp_path / "t.json")]) == 0
    assert json.loads((tmp_path / "t.json").read_text())["entries"][0]["coll"] == "all_reduce"
    with pytest.raises(ValueError):
        tune.build_table({"ll": ll, "p2p": dict(p2p, nranks=4)})


def test_derived_counters_parser_and_evaluation(tmp_path, capsys):
    from rocm_systems_b200.tools import counters, roofline

    ast = counters.parse("max(1, (a.b + 2 * -c) / 4) - select(d, 10, 20)")
    assert counters.evaluate(ast, {"a.b": 10, "c": 1, "d": 0}) == 2.0 - 20
    assert counters.evaluate(ast, {"a.b": 2, "c": 1, "d": 5}) == 1.0 - 10
    assert sorted(set(counters.identifiers(ast))) == ["a.b", "c", "d"]
    assert counters.evaluate(counters.parse("1e3 / 0"), {}) != counters.evaluate(counters.parse("1e3 / 0"), {})   # NaN, not an exception
    for bad in ("1 +", "foo(1)", "(1", "1 $ 2", "1 2"):
        with pytest.raises(counters.ParseError):
            counters.parse(bad)
    cs = counters.CounterSet.load()
    need = cs.required_metrics()
    assert "dram__bytes_read.sum" in need and "gpu__time_duration.sum" in need and not any(n.startswith(("peak.", "arg.")) for n in need)
    k = roofline.parse_ncu_csv(NCU_CSV)[1]     # the GEMM row: 1000 us, 200 + 134 MB
    vals = cs.evaluate(k.raw, {"hbm_gbs": 6541.5, "bf16_tflops": 1601.7}, {"flops": 2 * 8192.0 ** 3})
    assert abs(vals["hbm_gbs"] - 334.0) < 1e-6 and abs(vals["tflops"] - 1099.5) < 0.1 and abs(vals["bf16_fraction"] - 0.6865) < 1e-3
    assert vals["tensor_active_pct"] == 90 and vals["reread_factor"] is None          # arg.bytes was not given
    with pytest.raises(ValueError):
        counters.CounterSet([{"name": "x", "expression": "1"}, {"name": "x", "expression": "2"}])
    (tmp_path / "raw.csv").write_text(NCU_CSV)
    (tmp_path / "p.json").write_text(json.dumps({"hbm_gbs": 6541.5, "bf16_tflops": 1601.7}))
    assert counters.main([str(tmp_path / "raw.csv"), "--peaks", str(tmp_path / "p.json"), "--arg", "flops=1.0995e12"]) == 0
    out = capsys.readouterr().out
    assert "gemmKernel" in out and "bf16_fraction" in out
    assert counters.main(["--list"]) == 0


def test_tracing_overhead_harness(tmp_path):
    from rocm_systems_b200.bench import prof_overhead

    child = "from rocm_systems_b200.utils import markers\nimport time\nwith markers.range('w'):\n    time.sleep(0.05)\n"
    os.environ.setdefault("PYTHONPATH", str(ROOT))
    res = prof_overhead.measure([sys.executable, "-c", child], {"markers": "--marker-trace"}, repeat=2)
    assert len(res["baseline_s"]) == 2 and res["configs"]["markers"]["median_s"] > 0
    prof_overhead.store(str(tmp_path / "o.db"), res)
    import sqlite3

    rows = sqlite3.connect(str(tmp_path / "o.db")).execute("select config, repeat from overhead").fetchall()
    assert rows == [("markers", 2)]


def test_telemetry_groups_and_diagnostics(fake_nvml):
    out = _py("""
from rocm_systems_b200.tools import telemetry
t = telemetry.Telemetry()
t.create_group('pair', [0, 2]); t.create_field_group('thermal', ['temp', 'power'])
try:
    t.create_group('bad', [9]); raise SystemExit('bad group accepted')
except ValueError:
    pass
t.watch('pair', 'thermal', period_ms=20, keep=10)
assert t.devices == [0, 2] and t.fields == ['temp', 'power']
t.stop()
d = {r['device']: r for r in t.diagnose(1)}
assert d[0]['pass'] and not d[2]['pass']
failed = [c['check'] for c in d[2]['checks'] if not c['pass']]
assert failed == ['nvlink_errors'], failed
print('ok')
""", {"B200SMI_NVML_LIBRARY": fake_nvml, "FAKE_NVML_GPUS": "4", "FAKE_NVML_LINK_ERRORS": "2"})
    assert "ok" in out
    e = dict(os.environ, PYTHONPATH=str(ROOT), B200SMI_NVML_LIBRARY=fake_nvml, FAKE_NVML_GPUS="2", FAKE_NVML_ECC="1")
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.telemetry", "diag"], env=e, capture_output=True, text=True, timeout=120)
    assert p.returncode == 1 and "GPU 1: FAIL" in p.stdout and "GPU 0: PASS" in p.stdout, p.stdout + p.stderr


def test_roofline_and_counters_on_a_recorded_capture(capsys):
    """A recorded Nsight Compute raw page of the tcgen05 GEMM (4096^3 bf16 on a B200), reduced to the
    columns the tools read: analysis needs no GPU, as with the reference's recorded workloads."""
    from rocm_systems_b200.tools import counters, roofline

    path = str(ROOT / "tests" / "fixtures" / "gemm_tcgen05_ncu_raw.csv")
    ks = roofline.read_ncu(path)
    assert len(ks) >= 1 and "gemmKernel" in ks[0].name
    k = ks[0]
    assert 50e3 < k.duration_ns < 500e3 and k.counters["tensor_pct"] > 50 and k.counters["registers"] > 0
    k.flops = 2 * 4096.0 ** 3
    peaks = {"hbm_gbs": 6541.5, "bf16_tflops": 1601.7, "source": "measured"}
    assert roofline.classify(k, peaks) == "compute" and 0.5 < k.tflops / peaks["bf16_tflops"] < 1.1
    vals = counters.CounterSet.load().evaluate(k.raw, peaks, {"flops": k.flops, "bytes": 3 * 4096 * 4096 * 2})
    assert vals["tensor_active_pct"] > 50 and 0.9 < vals["reread_factor"] < 2.0 and vals["arithmetic_intensity"] > 500
    assert roofline.main([path, "--peaks", "/nonexistent.json", "--flops", "gemm=1.374e11"]) == 0
    assert "of nominal" in capsys.readouterr().out


def test_tool_registration_is_once_under_concurrent_first_use(tmp_path):
    """Many threads make the first API call at once: the dispatch table is built once, the tool is
    configured once (listing it twice does not load it twice) and no call is lost."""
    from rocm_systems_b200.utils import build

    tool = build.build_sample_tool()
    out = tmp_path / "tool.txt"
    _py("""
import ctypes, threading
from rocm_systems_b200 import _lib
lib = _lib.load()
start = threading.Barrier(16)
def work():
    v = ctypes.c_int()
    start.wait()
    for _ in range(50):
        assert lib.ncclGetVersion(ctypes.byref(v)) == 0 and v.value == 22005
ts = [threading.Thread(target=work) for _ in range(16)]
[t.start() for t in ts]; [t.join() for t in ts]
""", {"B200COLL_TOOL_LIBRARIES": f"{tool}:{tool}", "B200COLL_SAMPLE_TOOL_OUTPUT": str(out)})
    assert "ncclGetVersion calls=800" in out.read_text()


def test_output_validators(tmp_path):
    from rocm_systems_b200.tools import tracedb, validate

    (tmp_path / "t.100_kernel_trace.csv").write_text(KERNEL_CSV)
    (tmp_path / "t.rank0.csv").write_text(COLL_CSV)
    (tmp_path / "t.markers.100.csv").write_text(MARK_CSV)
    dbp = str(tmp_path / "t.db")
    with tracedb.TraceDB(dbp) as db:
        for p in sorted(tmp_path.glob("t.*csv")):
            db.import_csv(str(p))
        db.to_perfetto(str(tmp_path / "t.json"))
    assert validate.check_perfetto(str(tmp_path / "t.json"), categories=["kernel", "collective", "MARKER_API"], names=["gemmKernel"], min_slices=8) == []
    errs = validate.check_perfetto(str(tmp_path / "t.json"), categories=["memcpy"], counters=["gpu_power"], min_slices=100)
    assert len(errs) == 3
    assert validate.check_db(dbp, ["kernel_dispatch:3", "collective:2", "top_kernels:2"]) == []
    assert validate.check_db(dbp, ["kernel_dispatch:4", "nope"]) == ["kernel_dispatch: 3 rows, expected at least 4", "no table or view 'nope'"]
    assert validate.check_csv(str(tmp_path / "t.rank0.csv"), ["Device_Us", "AlgBw_GBps"], ["ncclAllReduce"]) == []
    assert validate.check_csv(str(tmp_path / "t.rank0.csv"), ["Nope"], ["ncclBroadcast"], min_rows=5) != []
    # partially overlapping slices on one track are flagged
    bad = {"traceEvents": [{"ph": "X", "pid": 1, "tid": "a", "name": "x", "ts": 0, "dur": 10}, {"ph": "X", "pid": 1, "tid": "a", "name": "y", "ts": 5, "dur": 10}]}
    (tmp_path / "bad.json").write_text(json.dumps(bad))
    assert any("overlap" in e for e in validate.check_perfetto(str(tmp_path / "bad.json")))
    assert validate.main(["db", dbp, "--table", "region:1"]) == 0
    # arrows: the two collective calls point at their device intervals; a lone or backward arrow is flagged
    assert validate.check_perfetto(str(tmp_path / "t.json"), min_flows=2) == []
    assert validate.check_perfetto(str(tmp_path / "t.json"), min_flows=3) == ["2 arrows, expected at least 3"]
    lone = {"traceEvents": [{"ph": "s", "id": 1, "pid": 1, "tid": "a", "ts": 5}, {"ph": "s", "id": 2, "pid": 1, "tid": "a", "ts": 9},
                            {"ph": "f", "id": 2, "pid": 1, "tid": "b", "ts": 3}]}
    (tmp_path / "lone.json").write_text(json.dumps(lone))
    errs = validate.check_perfetto(str(tmp_path / "lone.json"))
    assert any("without their other end" in e for e in errs) and any("back in time" in e for e in errs)
    # the causal profiler's output
    coz = tmp_path / "e.coz"
    coz.write_text("startup\ttime=1\nexperiment\tselected=cpu_slow_func\tspeedup=0.20\tduration=800\tselected-samples=5\treal-duration=1000\n"
                   "throughput-point\tname=iteration\tdelta=10\nruntime\ttime=2\n")
    assert validate.check_causal(str(coz), 1, ["slow"], ["iteration"]) == []
    errs = validate.check_causal(str(coz), 3, ["fast"], ["other"])
    assert len(errs) == 3
    coz.write_text("experiment\tselected=f\tspeedup=0.20\tduration=1200\tselected-samples=5\treal-duration=1000\n")
    assert any("duration 1200 of 1000" in e for e in validate.check_causal(str(coz)))
    assert validate.main(["causal", str(coz)]) == 1


def test_telemetry_policy_events_over_http(fake_nvml):
    out = _py("""
import json, time, urllib.request
from rocm_systems_b200.tools import telemetry
t = telemetry.Telemetry()
srv = telemetry.serve(t, '127.0.0.1', 0)
url = 'http://127.0.0.1:%d' % srv.server_address[1]
get = lambda p: urllib.request.urlopen(url + p, timeout=10).read().decode()
get('/api/policy/set?dev=0&field=power&threshold=250&direction=above')     # watts; the stand-in ramps by 10 W per read
t.start(devices=[0], fields=['power'], period_ms=20, keep=100)
deadline = time.time() + 5
ev = []
while time.time() < deadline and not ev:
    time.sleep(0.1)
    ev = json.loads(get('/api/policy/events'))
assert ev and ev[0]['device'] == 0 and ev[0]['field'] == 'power' and ev[0]['value'] > 250 and ev[0]['direction'] == 'above'
try:
    get('/api/policy/set?dev=0&field=nope&threshold=1'); raise SystemExit('bad field accepted')
except urllib.error.HTTPError as e:
    assert e.code == 400
srv.shutdown(); t.stop()
print('ok')
""", {"B200SMI_NVML_LIBRARY": fake_nvml, "FAKE_NVML_GPUS": "2", "FAKE_NVML_RAMP": "1"})
    assert "ok" in out


def test_perfetto_export_draws_launch_arrows(tmp_path):
    """A runtime API record and the kernel with the same correlation id are joined by a flow; a kernel without a call record
    and a marker range are not."""
    from rocm_systems_b200.tools import tracedb

    (tmp_path / "t.100_kernel_trace.csv").write_text(KERNEL_CSV)
    (tmp_path / "t.100_cuda_api_trace.csv").write_text(
        '"Domain","Function","Process_Id","Thread_Id","Correlation_Id","Start_Timestamp","End_Timestamp"\n'
        '"CUDA_RUNTIME_API","cudaLaunchKernel",100,101,1,800,850\n"CUDA_RUNTIME_API","cudaLaunchKernel",100,101,3,9000,9100\n'
        '"CUDA_RUNTIME_API","cudaMalloc",100,101,0,100,200\n')
    (tmp_path / "t.markers.100.csv").write_text(MARK_CSV)
    with tracedb.TraceDB(str(tmp_path / "t.db")) as db:
        for p in sorted(tmp_path.glob("t.*csv")):
            db.import_csv(str(p))
        db.to_perfetto(str(tmp_path / "t.json"))
    ev = json.loads((tmp_path / "t.json").read_text())["traceEvents"]
    starts = {e["id"]: e for e in ev if e["ph"] == "s"}
    ends = {e["id"]: e for e in ev if e["ph"] == "f"}
    assert len(starts) == len(ends) == 2 and all(e["bp"] == "e" for e in ends.values())
    pairs = sorted((starts[i]["ts"], ends[i]["ts"], starts[i]["tid"], ends[i]["tid"]) for i in starts)
    assert pairs == [(0.8, 1.0, "CUDA_RUNTIME_API 101", "gpu0 stream 7"), (9.0, 9.5, "CUDA_RUNTIME_API 101", "gpu0 stream 7")]


def test_tracedb_postprocessing_filters(tmp_path):
    """Exclusion by regex, short kernel names and the collection window (rocprofv3's --kernel-exclude-regex,
    --truncate-kernels and --collection-period, applied to the imported trace)."""
    from rocm_systems_b200.tools import tracedb

    assert tracedb.TraceDB.short_kernel_name("void b200::gemm::gemmKernel<256, b200::gemm::PlainPolicy<256> >(b200::gemm::Params, int)") == "gemmKernel"
    assert tracedb.TraceDB.short_kernel_name("rmsnorm") == "rmsnorm"
    assert tracedb.TraceDB.short_kernel_name("void at::native::(anonymous namespace)::vectorized_elementwise_kernel<4, Foo>(int)") == "vectorized_elementwise_kernel"
    csv_text = KERNEL_CSV.replace('"gemmKernel<Cfg>",1,', '"void ns::gemmKernel<128, P<128> >(Params)",1,').replace('"gemmKernel<Cfg>",2,', '"void ns::gemmKernel<256, P<256> >(Params)",2,')
    (tmp_path / "t.100_kernel_trace.csv").write_text(csv_text)
    (tmp_path / "t.rank0.csv").write_text(COLL_CSV)
    with tracedb.TraceDB(str(tmp_path / "a.db")) as db:
        for p in sorted(tmp_path.glob("t.*csv")):
            db.import_csv(str(p))
        assert len(db.summary()["kernels"]) == 3                               # two instantiations and rmsnorm
        assert db.truncate_kernel_names() == 2
        top = db.summary()["kernels"][0]
        assert top["name"] == "gemmKernel" and top["calls"] == 2               # the instantiations aggregate
        assert db.drop_kernels("^rms") == 1
        assert [k["name"] for k in db.summary()["kernels"]] == ["gemmKernel"]
    with tracedb.TraceDB(str(tmp_path / "b.db")) as db:
        for p in sorted(tmp_path.glob("t.*csv")):
            db.import_csv(str(p))
        # first record starts at 900 ns (a collective's host entry); keep [900 + 5000, 900 + 5000 + 4000) ns
        gone = db.keep_window(0.005, 0.004)
        names, rows = db.query("select start_ns from kernels order by start_ns")
        assert rows == [(6000,), (9500,)] and gone == 1 + 2 + 2      # one kernel, both collectives and their two API regions


def test_tracedb_iteration_ranges_domains_groups_and_units(tmp_path):
    """Launch numbers per kernel (--kernel-iteration-range), statistics per domain and over unions of domains
    (--summary-per-domain, --summary-groups) and the unit of the time columns (--summary-units)."""
    from rocm_systems_b200.tools import tracedb

    T = tracedb.TraceDB
    assert T.parse_iteration_ranges(["[1-3]", "5", "[8-]", "[10,12-13]"]) == [(1, 3), (5, 5), (8, None), (10, 10), (12, 13)]
    with pytest.raises(ValueError):
        T.parse_iteration_ranges(["[a-3]"])
    (tmp_path / "t.100_kernel_trace.csv").write_text(KERNEL_CSV)
    (tmp_path / "t.rank0.csv").write_text(COLL_CSV)
    (tmp_path / "t.markers.100.csv").write_text(MARK_CSV)
    with T(str(tmp_path / "a.db")) as db:
        for p in sorted(tmp_path.glob("t.*csv")):
            db.import_csv(str(p))
        doms = db.domain_summaries(top=5, groups=["KERNEL_DISPATCH|COLLECTIVE", "MARKER_.*"])
        assert set(doms["domains"]) == {"KERNEL_DISPATCH", "COLLECTIVE", "MARKER_API", "B200COLL_API"}
        k = doms["domains"]["KERNEL_DISPATCH"]
        assert [r["name"] for r in k] == ["gemmKernel<Cfg>", "rmsnorm"] and k[0]["calls"] == 2 and k[0]["total_ns"] == 7000
        assert k[0]["min_ns"] == 3000 and k[0]["max_ns"] == 4000 and k[0]["percent"] == pytest.approx(100 * 7000 / 7500)
        union = doms["groups"]["KERNEL_DISPATCH|COLLECTIVE"]
        assert [(r["domain"], r["name"]) for r in union] == [("COLLECTIVE", "ncclAllReduce"), ("KERNEL_DISPATCH", "gemmKernel<Cfg>"), ("KERNEL_DISPATCH", "rmsnorm")]
        assert union[0]["percent"] == pytest.approx(100 * 18000 / 25500)
        assert [r["name"] for r in doms["groups"]["MARKER_.*"]] == ["step 0"]
        scaled = tracedb.scale_units(doms, "usec")
        row = scaled["domains"]["KERNEL_DISPATCH"][0]
        assert "total_ns" not in row and row["total_usec"] == pytest.approx(7.0) and row["mean_usec"] == pytest.approx(3.5) and row["calls"] == 2
        assert tracedb.scale_units(doms, "nsec") is doms
        import io

        buf = io.StringIO()
        tracedb.print_summary(dict(db.summary(), **scaled), file=buf)
        assert "== DOMAIN KERNEL_DISPATCH ==" in buf.getvalue() and "== GROUP MARKER_.* ==" in buf.getvalue() and "total_usec" in buf.getvalue()
        # second launch of every kernel only: gemmKernel's second, nothing of rmsnorm (launched once)
        assert db.keep_kernel_iterations([(2, 2)]) == 2
        assert db.query("select name, start_ns from kernels")[1] == [("gemmKernel<Cfg>", 6000)]


def test_tracedb_diff_names_what_got_slower(tmp_path, capsys):
    """Two traces of one program: the slower kernel leads the table, a kernel that exists on one side only is listed, the
    threshold hides what did not move, and --fail-above turns the comparison into a check."""
    from rocm_systems_b200.tools import tracedb

    slow = KERNEL_CSV.replace(",6000,9000,", ",6000,12000,").replace('"rmsnorm",3,9500,10000', '"rmsnorm2",3,12500,13000')
    for name, text in (("a", KERNEL_CSV), ("b", slow)):
        d = tmp_path / name
        d.mkdir()
        (d / "t.100_kernel_trace.csv").write_text(text)
        (d / "t.rank0.csv").write_text(COLL_CSV)
        assert tracedb.main(["import", str(d / "t.100_kernel_trace.csv"), str(d / "t.rank0.csv"), "-o", str(d / "t.db")]) == 0
    capsys.readouterr()
    with tracedb.TraceDB(str(tmp_path / "a" / "t.db")) as x, tracedb.TraceDB(str(tmp_path / "b" / "t.db")) as y:
        rows = tracedb.diff(x, y)
        assert [r["name"] for r in rows[:3]] == ["gemmKernel<Cfg>", "rmsnorm", "rmsnorm2"] or [r["name"] for r in rows[:3]] == ["gemmKernel<Cfg>", "rmsnorm2", "rmsnorm"]
        g = rows[0]
        assert g["base_total_ns"] == 7000 and g["total_ns"] == 10000 and g["change_percent"] == pytest.approx(100 * 3000 / 7000) and g["calls"] == 2
        assert g["share_of_base_percent"] == pytest.approx(100 * 3000 / 25500)
        gone = next(r for r in rows if r["name"] == "rmsnorm")
        assert gone["calls"] == 0 and gone["change_percent"] == -100.0
        new = next(r for r in rows if r["name"] == "rmsnorm2")
        assert new["base_calls"] == 0 and new["change_percent"] == float("inf")
        assert {r["name"] for r in tracedb.diff(x, y, min_change=50.0)} == {"rmsnorm", "rmsnorm2"}        # the collective did not move; the GEMM moved 43 %
        assert [r["name"] for r in tracedb.diff(x, y, domains=["COLLECTIVE"])] == ["ncclAllReduce"]
    assert tracedb.main(["diff", str(tmp_path / "a" / "t.db"), str(tmp_path / "b" / "t.db"), "--fail-above", "20"]) == 0
    out = capsys.readouterr().out
    assert "gemmKernel<Cfg>" in out and "base_total_usec" in out and "(+11.76 %)" in out                    # 25500 -> 28500 ns
    assert tracedb.main(["diff", str(tmp_path / "a" / "t.db"), str(tmp_path / "b" / "t.db"), "--fail-above", "5", "--json"]) == 1
    assert json.loads(capsys.readouterr().out)["change_percent"] == pytest.approx(100 * 3000 / 25500)
    assert tracedb.main(["summary", str(tmp_path / "a" / "t.db"), "--per-domain", "--units", "usec"]) == 0
    assert "== DOMAIN KERNEL_DISPATCH ==" in capsys.readouterr().out


def test_prof_launcher_summary_and_environment_options(tmp_path, capsys):
    """--kokkos-trace, --preload and --echo reach the environment of the command; --output-config records the pass."""
    from rocm_systems_b200.tools import prof
    from rocm_systems_b200.utils import build

    lib = build.build_kokkosp()
    a = prof.parser().parse_args(["--kokkos-trace", "--preload", "/x/liba.so", "--preload", "/x/libb.so", "--summary-groups", "A|B", "--summary-units", "msec",
                                  "--kernel-iteration-range", "[2-4]", "--collection-period", "1:2", "--collection-period-unit", "sec", "--", "true"])
    env = prof.build_env(a, str(tmp_path / "t"))
    assert env["KOKKOS_TOOLS_LIBS"].split(";")[0] == str(lib)
    assert env["LD_PRELOAD"].split(":")[:2] == ["/x/liba.so", "/x/libb.so"]
    assert a.summary_groups == ["A|B"] and a.summary_units == "msec" and a.kernel_iteration_range == ["[2-4]"] and a.collection_period_unit == "sec"
    rc = prof.main(["--marker-trace", "--echo", "--output-config", "-d", str(tmp_path), "-o", "run", "--", sys.executable, "-c", "pass"])
    assert rc == 0
    err = capsys.readouterr().err
    assert "B200COLL_TRACE=1" in err and "-c pass" in err
    cfg = json.loads((tmp_path / "run_config.json").read_text())
    assert cfg["marker_trace"] is True and cfg["echo"] is True and cfg["command"][-2:] == ["-c", "pass"]


def test_prof_launcher_applies_filters(tmp_path):
    from rocm_systems_b200.tools import prof

    a = prof.parser().parse_args(["--kernel-trace", "--kernel-exclude-regex", "rms", "--truncate-kernels", "--collection-period", "0:100", "--", "true"])
    assert a.kernel_exclude_regex == "rms" and a.truncate_kernels and a.collection_period == "0:100"


def test_telemetry_device_events_over_http_and_prometheus(fake_nvml):
    out = _py("""
import json, time, urllib.request
from rocm_systems_b200.tools import telemetry
t = telemetry.Telemetry()
srv = telemetry.serve(t, '127.0.0.1', 0)
url = 'http://127.0.0.1:%d' % srv.server_address[1]
get = lambda p: urllib.request.urlopen(url + p, timeout=10).read().decode()
t.start_event_listener()
deadline = time.time() + 5
ev = []
while time.time() < deadline and len(ev) < 2:
    time.sleep(0.1)
    ev = json.loads(get('/api/events'))
assert [(e['device'], e['type'], e['data']) for e in ev] == [(1, 'xid', 79), (0, 'ecc_double_bit', 2)], ev
text = get('/metrics')
assert 'b200_device_events_total{gpu="1",type="xid"} 1' in text and 'b200_device_events_total{gpu="0",type="ecc_double_bit"} 1' in text
srv.shutdown(); t.stop()
print('ok')
""", {"B200SMI_NVML_LIBRARY": fake_nvml, "FAKE_NVML_GPUS": "2", "FAKE_NVML_EVENTS": "1:8:79,0:2:2"})
    assert "ok" in out


def test_hang_dump_reports_stacks_and_communicator_state(tmp_path):
    """After the deadline: every thread's stack and each communicator's error text; a kick postpones it; exit_after ends
    the process with 124."""
    out = _py("""
import io, sys, threading, time
from rocm_systems_b200.utils import hang_dump
class Fake:
    rank, nranks = 2, 8
    def async_error(self): return 6
    def last_error(self): return 'wait BARRIER for rank 5 gave up: expected 12, saw 11'
buf = io.StringIO()
def stuck_worker():
    time.sleep(2)
threading.Thread(target=stuck_worker, daemon=True).start()
hang_dump.arm(0.3, comms=[Fake()], file=sys.stdout)
time.sleep(0.2); hang_dump.kick(); time.sleep(0.2)      # 0.4 s in, but kicked at 0.2: nothing yet
print('QUIET' if True else '')
time.sleep(0.4)
hang_dump.disarm()
print('END')
""")
    quiet, rest = out.split("QUIET", 1)
    assert "hang_dump" not in quiet
    assert "no progress for 0 s" in rest and "stuck_worker" in rest and "rank 2/8: async error 6" in rest and "expected 12, saw 11" in rest
    p = subprocess.run([sys.executable, "-c", "import time\nfrom rocm_systems_b200.utils import hang_dump\nhang_dump.arm(0.2, exit_after=True)\ntime.sleep(5)"],
                       env=dict(os.environ, PYTHONPATH=str(ROOT)), capture_output=True, text=True, timeout=60)
    assert p.returncode == 124 and "hang_dump" in p.stderr


def test_counters_collection_command_asks_for_exactly_the_needed_metrics(capsys):
    """--collect builds a bounded Nsight Compute capture (clocks untouched, one kernel pattern, few launches) for the raw
    metrics the chosen definitions read, and refuses an unbounded launch count."""
    from rocm_systems_b200.tools import counters

    rc = counters.main(["--collect", "-k", "gemmPairKernel", "-c", "2", "--counter", "tensor_active_pct", "--counter", "hbm_gbs", "--print-command",
                        "--", "python", "-m", "rocm_systems_b200.bench.kernel_cases", "--case", "gemm"])
    assert rc == 0
    line = capsys.readouterr().out.strip().split()
    assert line[0] == "ncu" and line[1:3] == ["--clock-control", "none"]
    metrics = line[line.index("--metrics") + 1].split(",")
    assert sorted(metrics) == ["dram__bytes_read.sum", "dram__bytes_write.sum", "gpu__time_duration.sum", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active"]
    assert line[line.index("-c") + 1] == "2" and line[line.index("-k") + 1] == "regex:gemmPairKernel"
    assert line[-5:] == ["python", "-m", "rocm_systems_b200.bench.kernel_cases", "--case", "gemm"]
    with pytest.raises(SystemExit):
        counters.main(["--collect", "-c", "500", "--print-command", "--", "true"])
    with pytest.raises(SystemExit):
        counters.main(["--collect", "--counter", "no_such_counter", "--print-command", "--", "true"])


ANALYZE_COLS = [
    ("Kernel Name", ""), ("gpu__time_duration.sum", "us"), ("dram__bytes_read.sum", "Mbyte"), ("dram__bytes_write.sum", "Mbyte"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "%"), ("gpu__compute_memory_throughput.avg.pct_of_peak_sustained_elapsed", "%"),
    ("sm__throughput.avg.pct_of_peak_sustained_elapsed", "%"), ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "%"),
    ("sm__cycles_active.avg", "cycle"), ("sm__cycles_elapsed.avg", "cycle"), ("lts__t_sector_hit_rate.pct", "%"),
    ("launch__grid_size", ""), ("launch__block_size", ""), ("launch__waves_per_multiprocessor", ""), ("launch__registers_per_thread", "register/thread"),
    ("smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio", "inst"),
    ("smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio", "inst"),
    ("smsp__average_warps_issue_stalled_selected_per_issue_active.ratio", "inst"),
]
ANALYZE_ROWS = [
    # a streaming kernel near the memory ceiling, a tensor-core kernel, and a 16-CTA kernel that mostly waits at barriers
    ["streamKernel", "100", "300", "300", "78", "80", "20", "0", "95000", "100000", "2", "4096", "256", "6.9", "32", "9.0", "0.2", "1.0"],
    ["mmaKernel", "1000", "200", "134", "5", "30", "85", "82", "99000", "100000", "70", "148", "192", "1.0", "168", "1.5", "0.4", "1.0"],
    ["waitKernel", "700", "147", "182", "6", "6", "1", "0", "10000", "100000", "20", "16", "512", "0.11", "128", "20.4", "30.6", "1.0"],
]


def _analyze_csv() -> str:
    q = lambda cells: ",".join(f'"{c}"' for c in cells)  # noqa: E731
    return "\n".join([q([c for c, _ in ANALYZE_COLS]), q([u for _, u in ANALYZE_COLS])] + [q(r) for r in ANALYZE_ROWS]) + "\n"


def test_counter_analysis_panels_stalls_and_verdicts(tmp_path, capsys):
    from rocm_systems_b200.tools import counters, roofline

    cs = counters.CounterSet.load()
    assert {d.get("panel") for d in cs.defs} <= set(counters.PANELS)           # every definition sits in a known panel
    items = counters.analyze(cs, roofline.parse_ncu_csv(_analyze_csv()), {"hbm_gbs": 6650.0, "bf16_tflops": 1600.0}, {})
    by = {it["kernel"]: it for it in items}
    assert by["streamKernel"]["verdict"].startswith("memory bound")            # 600 MB in 100 us = 6 TB/s of 6.65
    assert by["mmaKernel"]["verdict"].startswith("compute bound")
    assert by["waitKernel"]["verdict"].startswith("under-filled") and "barrier" in by["waitKernel"]["verdict"]
    st = by["waitKernel"]["stalls"]
    assert [s["reason"] for s in st] == ["barrier", "long_scoreboard"]         # ranked; "selected" (issuing) is not a stall
    mem = {r["name"]: r["value"] for r in by["streamKernel"]["panels"]["memory"]}
    assert abs(mem["hbm_gbs"] - 6000) < 1e-6 and abs(mem["dram_read_mb"] - 300) < 1e-9
    sol = {r["name"]: r["value"] for r in by["waitKernel"]["panels"]["speed_of_light"]}
    assert abs(sol["sm_active_pct"] - 10.0) < 1e-9
    assert "compute" not in by["waitKernel"]["panels"] or all(r["name"] != "ipc_active" for r in by["waitKernel"]["panels"]["compute"])  # inputs absent: left out
    # the command line prints the same analysis
    (tmp_path / "raw.csv").write_text(_analyze_csv())
    (tmp_path / "p.json").write_text('{"hbm_gbs": 6650.0, "bf16_tflops": 1600.0}')
    assert counters.main([str(tmp_path / "raw.csv"), "--analyze", "--peaks", str(tmp_path / "p.json")]) == 0
    text = capsys.readouterr().out
    assert "== waitKernel" in text and "[stalls" in text and "under-filled" in text and "[memory]" in text
    assert counters.main([str(tmp_path / "raw.csv"), "--list-kernels"]) == 0
    listing = capsys.readouterr().out.splitlines()
    assert len(listing) == 3 and all(" x " in l and l.rstrip().endswith(("streamKernel", "mmaKernel", "waitKernel")) for l in listing)
    # and as one self-contained page
    assert counters.main([str(tmp_path / "raw.csv"), "--analyze", "--peaks", str(tmp_path / "p.json"), "--html", str(tmp_path / "a.html")]) == 0
    page = (tmp_path / "a.html").read_text()
    assert page.startswith("<!doctype html>") and page.count("<h2 id=") == 3 and "under-filled" in page and "<script" not in page and "http" not in page
    assert 'href="#k2"' in page and "stalls (stalled warps per issued instruction)" in page and 'class="bar"' in page
    evil = counters.html_report([{"kernel": "k<img src=x>", "verdict": "a & b", "panels": {}, "stalls": []}])
    assert "<img" not in evil and "k&lt;img src=x&gt;" in evil and "a &amp; b" in evil


def test_counter_collection_leaves_a_machine_description(tmp_path, capsys, monkeypatch):
    """--collect with the Nsight Compute run and the report reader replaced: the capture is followed by a sysinfo file (or,
    where the machine cannot be described, by a note), never by a failure."""
    import subprocess as sp

    from rocm_systems_b200.tools import counters, roofline

    calls = []
    monkeypatch.setattr(sp, "call", lambda cmd, **k: calls.append(cmd) or 0)
    monkeypatch.setattr(roofline, "read_ncu", lambda path: roofline.parse_ncu_csv(_analyze_csv()))
    (tmp_path / "p.json").write_text('{"hbm_gbs": 6650.0, "bf16_tflops": 1600.0}')
    out = tmp_path / "cap"
    rc = counters.main(["--collect", "--counter", "hbm_gbs", "-k", "stream", "-c", "1", "-o", str(out), "--peaks", str(tmp_path / "p.json"), "--", "python", "x.py"])
    text = capsys.readouterr()
    assert rc == 0 and calls and calls[0][0] == "ncu" and "--clock-control" in calls[0] and "streamKernel" in text.out
    info = tmp_path / "cap_sysinfo.json"
    assert info.exists() or "no sysinfo file" in text.err
    if info.exists():
        doc = json.loads(info.read_text())
        assert doc["command"] == ["python", "x.py"] and doc["counters"] == ["hbm_gbs"] and "host" in doc


def test_profiler_launcher_counter_collection(tmp_path, capsys):
    """``prof --pmc``: the Nsight Compute line asks for exactly the raw metrics of the chosen counters (bounded, clocks
    untouched), and a capture becomes one row per (launch, counter)."""
    import csv as _csv

    from rocm_systems_b200.tools import counters, prof, roofline

    rc = prof.main(["--pmc", "hbm_gbs", "tensor_active_pct", "--pmc-kernel", "gemm", "--pmc-count", "2", "--pmc-dry-run", "-d", str(tmp_path), "--", "python", "x.py"])
    line = capsys.readouterr().out.strip()
    assert rc == 0 and line.startswith("ncu --clock-control none --metrics ") and line.endswith("-k regex:gemm python x.py") and " -c 2 " in line
    metrics = line.split("--metrics ")[1].split(" ")[0].split(",")
    assert sorted(metrics) == ["dram__bytes_read.sum", "dram__bytes_write.sum", "gpu__time_duration.sum", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active"]
    assert prof.main(["--pmc", "no_such_counter", "--pmc-dry-run", "-d", str(tmp_path), "--", "true"]) == 2
    assert prof.main(["--pmc", "hbm_gbs", "--pmc-count", "500", "--pmc-dry-run", "-d", str(tmp_path), "--", "true"]) == 2
    capsys.readouterr()
    assert prof.main(["--list-pmc"]) == 0 and "hbm_gbs" in capsys.readouterr().out
    cs = counters.CounterSet.load()
    n = prof.write_counter_collection(cs, roofline.parse_ncu_csv(_analyze_csv()), {"hbm_gbs": 6650.0, "bf16_tflops": 1600.0}, str(tmp_path / "cc.csv"))
    rows = list(_csv.DictReader(open(tmp_path / "cc.csv")))
    assert n == len(rows) and {r["Kernel_Name"] for r in rows} == {"streamKernel", "mmaKernel", "waitKernel"}
    got = {(r["Kernel_Name"], r["Counter_Name"]): float(r["Counter_Value"]) for r in rows}
    assert abs(got[("streamKernel", "hbm_gbs")] - 6000) < 1e-3 and got[("mmaKernel", "tensor_active_pct")] == 82
    assert ("streamKernel", "tflops") not in got          # needs arg.flops: left out


def test_telemetry_group_management_and_saved_configuration(tmp_path, fake_nvml):
    """Device groups, field groups, a watch on a (group, field group) pair, the policy list, a device's links and a settings
    file that re-creates all of it in a second daemon: over HTTP and through the client command line."""
    out = _py(f"""
import json, io, contextlib, urllib.request, urllib.error
from rocm_systems_b200.tools import telemetry
t = telemetry.Telemetry()
srv = telemetry.serve(t, '127.0.0.1', 0)
url = 'http://127.0.0.1:%d' % srv.server_address[1]
def cli(*args):
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        assert telemetry.main(['client', '--url', url, *args]) == 0
    return json.loads(buf.getvalue())
assert cli('group-create', '--name', 'pair', '--devices', '1', '3') == {{'ok': True}}
assert cli('fieldgroup-create', '--name', 'thermal', '--fields', 'temp', 'power') == {{'ok': True}}
assert cli('group-list') == {{'all': [0, 1, 2, 3], 'pair': [1, 3]}}
assert cli('fieldgroup-list')['thermal'] == ['temp', 'power']
w = cli('watch', '--group', 'pair', '--fieldgroup', 'thermal', '--period-ms', '20')
assert w['devices'] == [1, 3] and w['fields'] == ['temp', 'power']
assert sorted(cli('latest')) == ['1', '3']
cli('policy-set', '--dev', '1', '--field', 'temp', '--threshold', '90', '--direction', 'above')
assert cli('policy-list') == [{{'device': 1, 'field': 'temp', 'threshold': 90.0, 'direction': 'above'}}]
topo = cli('topo', '--dev', '2')
assert [l['peer'] for l in topo] == [0, 1, 3] and topo[0]['type'] == 'NVLINK'
cli('config-save', '--path', r'{tmp_path}/cfg.json')
for bad in ('/api/group/create?name=x&devices=9', '/api/group/delete?name=all', '/api/watch?group=nope', '/api/fieldgroup/create?name=y&fields=bogus'):
    try:
        urllib.request.urlopen(url + bad, timeout=10); raise SystemExit('accepted ' + bad)
    except urllib.error.HTTPError as e:
        assert e.code == 400, bad
cli('group-delete', '--name', 'pair')
assert 'pair' not in cli('group-list')
srv.shutdown(); t.stop()
# a second daemon takes the saved settings
t2 = telemetry.Telemetry()
res = t2.config_load(r'{tmp_path}/cfg.json')
assert res['skipped'] == [] and t2.groups['pair'] == [1, 3] and t2.field_groups['thermal'] == ['temp', 'power'] and t2.config()['policies'][0]['threshold'] == 90.0
print('ok')
""", {"B200SMI_NVML_LIBRARY": fake_nvml, "FAKE_NVML_GPUS": "4"})
    assert "ok" in out


def test_kernels_renamed_after_the_marker_range_they_were_launched_in(tmp_path):
    from rocm_systems_b200.tools import tracedb

    api_csv = '''"Domain","Function","Process_Id","Thread_Id","Correlation_Id","Start_Timestamp","End_Timestamp"
"CUDA_RUNTIME_API","cudaLaunchKernel",100,100,1,600,610
"CUDA_RUNTIME_API","cudaLaunchKernel",100,100,2,700,710
"CUDA_RUNTIME_API","cudaLaunchKernel",100,200,3,800,810
'''
    marks = '''"Domain","Function","Process_Id","Thread_Id","Correlation_Id","Start_Timestamp","End_Timestamp","Depth"
"MARKER_API","step 0",100,100,1,500,20000,0
"MARKER_API","attention",100,100,2,650,750,1
'''
    (tmp_path / "t.100_kernel_trace.csv").write_text(KERNEL_CSV)
    (tmp_path / "t.100_runtime_trace.csv").write_text(api_csv)
    (tmp_path / "t.markers.100.csv").write_text(marks)
    with tracedb.TraceDB(str(tmp_path / "t.db")) as db:
        for p in sorted(tmp_path.glob("t.*csv")):
            db.import_csv(str(p))
        assert db.rename_kernels_by_marker() == 2
        _, rows = db.query("select name from kernels order by start_ns")
        # launched at 600 in "step 0"; at 700 inside the nested "attention"; the third from another thread, outside every range of that thread
        assert [r[0] for r in rows] == ["step 0", "attention", "rmsnorm"]
    # without API records the device start time decides (1000, 6000 and 9500 all lie inside "step 0" only)
    (tmp_path / "t.100_runtime_trace.csv").unlink()
    with tracedb.TraceDB(str(tmp_path / "u.db")) as db:
        for p in sorted(tmp_path.glob("t.*csv")):
            db.import_csv(str(p))
        assert db.rename_kernels_by_marker() == 3
        names, rows = db.query("select name, calls from top_kernels")
        assert rows == [("step 0", 3)]


def test_sweep_helpers_sizes_and_bus_bandwidth_factors():
    """The pure parts of the bandwidth sweep: size suffixes, and the bus-bandwidth factors of the rccl-tests harness
    (all_reduce 2(n-1)/n; all_gather, reduce_scatter, alltoall (n-1)/n; rooted collectives 1)."""
    from rocm_systems_b200.bench import coll_sweep as cs

    assert [cs.parse_size(s) for s in ("8", "64K", "1M", "8G", "1.5k")] == [8, 65536, 1 << 20, 8 << 30, 1536]
    assert cs.busbw_factor("all_reduce", 8) == 1.75 and cs.busbw_factor("all_reduce", 2) == 1.0
    for c in ("all_gather", "reduce_scatter", "alltoall"):
        assert cs.busbw_factor(c, 8) == 0.875 and cs.busbw_factor(c, 2) == 0.5
    assert cs.busbw_factor("broadcast", 8) == 1.0 and cs.busbw_factor("reduce", 4) == 1.0


def test_headline_summary_of_a_sweep(monkeypatch):
    """``headline.collectives_vs_nccl`` condenses sweep rows into what the benchmark line carries: the size ladder, per
    collective the ratio at every size, its minimum with the size it occurs at, the geometric mean and the bus bandwidth
    of both libraries at the largest size."""
    import math

    import torch

    from rocm_systems_b200.bench import coll_sweep, headline

    def fake_sweep(comm, colls, sizes, dt, send, recv, warmup, iters, nccl=True):
        rows = []
        for c in colls:
            for i, s in enumerate(sizes):
                ours = 10.0 + i
                rows.append({"coll": c, "bytes": s, "ours_us": ours, "nccl_us": ours * (0.5 if (c == "broadcast" and i == 1) else 2.0),
                             "ours_busbw": 100.0 + i, "nccl_busbw": 50.0 + i})
        return rows

    monkeypatch.setattr(coll_sweep, "sweep", fake_sweep)
    monkeypatch.setattr(torch, "empty", lambda *a, **k: type("T", (), {"normal_": lambda self: self})())

    class Comm:
        device = "cpu"

    out = headline.collectives_vs_nccl(Comm(), max_bytes=1 << 14, min_bytes=1 << 10, factor=4, colls=("all_reduce", "broadcast"))
    assert out["sizes_bytes"] == [1024, 4096, 16384]
    ar, bc = out["per_collective"]["all_reduce"], out["per_collective"]["broadcast"]
    assert ar["ratios"] == [2.0, 2.0, 2.0] and ar["min_ratio_vs_nccl"] == 2.0 and abs(ar["geomean_ratio_vs_nccl"] - 2.0) < 1e-12
    assert bc["min_ratio_vs_nccl"] == 0.5 and bc["min_ratio_at_bytes"] == 4096 and abs(bc["geomean_ratio_vs_nccl"] - math.exp((2 * math.log(2) + math.log(0.5)) / 3)) < 1e-12
    assert ar["busbw_gbs_at_max"] == 102.0 and ar["nccl_busbw_gbs_at_max"] == 52.0


def test_profiler_launcher_job_file(tmp_path):
    """``prof --input jobs.yaml``: every job is a pass of its own with the command line as defaults."""
    from rocm_systems_b200.tools import prof

    assert prof.job_argv({"kernel_trace": True, "coll-trace": False, "pmc": ["hbm_gbs", "tflops"], "top": 5, "kernel_include_regex": "gemm"}) == \
        ["--kernel-trace", "--pmc", "hbm_gbs", "tflops", "--top", "5", "--kernel-include-regex", "gemm"]
    (tmp_path / "jobs.yaml").write_text("jobs:\n  - marker_trace: true\n    stats: true\n  - marker_trace: true\n    output_format: [json]\n    output_file: second\n")
    child = "from rocm_systems_b200.utils import markers\nwith markers.range('phase'):\n    markers.mark('tick')\n"
    e = dict(os.environ, PYTHONPATH=str(ROOT))
    p = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.prof", "-i", str(tmp_path / "jobs.yaml"), "-d", str(tmp_path / "o"), "--",
                        sys.executable, "-c", child], env=e, capture_output=True, text=True, timeout=180)
    assert p.returncode == 0, p.stdout + p.stderr
    assert (tmp_path / "o" / "pass_0" / "trace.db").exists() and (tmp_path / "o" / "pass_0" / "trace_regions.csv").exists()
    assert (tmp_path / "o" / "pass_1" / "second.json").exists() and not (tmp_path / "o" / "pass_1" / "second.db").exists()
    assert "MARKER_API" in p.stdout and "pass 1" in p.stderr
    (tmp_path / "bad.json").write_text('{"jobs": []}')
    assert prof.main(["-i", str(tmp_path / "bad.json"), "--", "true"]) == 2
    # the plain-text form: one counter-collection pass per `pmc:` line
    (tmp_path / "in.txt").write_text("# two passes\npmc: hbm_gbs tflops\npmc: tensor_active_pct   # second\nkernel: gemmKernel rmsnorm\nrange: 0:1\n")
    assert prof.load_jobs(str(tmp_path / "in.txt")) == [{"pmc": ["hbm_gbs", "tflops"], "pmc_kernel": "gemmKernel|rmsnorm"},
                                                        {"pmc": ["tensor_active_pct"], "pmc_kernel": "gemmKernel|rmsnorm"}]
    (tmp_path / "none.txt").write_text("nothing here\n")
    assert prof.main(["-i", str(tmp_path / "none.txt"), "--", "true"]) == 2


def test_counter_comparison_of_two_captures(tmp_path, capsys):
    from rocm_systems_b200.tools import counters

    base = _analyze_csv()
    rows = [list(r) for r in ANALYZE_ROWS]
    rows[0][1] = "80"          # streamKernel: 100 us -> 80 us
    rows[1][7] = "90"          # mmaKernel: tensor pipe 82 -> 90 %
    q = lambda cells: ",".join(f'"{c}"' for c in cells)  # noqa: E731
    other = "\n".join([q([c for c, _ in ANALYZE_COLS]), q([u for _, u in ANALYZE_COLS])] + [q(r) for r in rows]) + "\n"
    (tmp_path / "a.csv").write_text(base)
    (tmp_path / "b.csv").write_text(other)
    (tmp_path / "p.json").write_text('{"hbm_gbs": 6650.0, "bf16_tflops": 1600.0}')
    assert counters.main([str(tmp_path / "a.csv"), "--compare", str(tmp_path / "b.csv"), "--peaks", str(tmp_path / "p.json"), "--json"]) == 0
    res = {r["kernel"]: {c["name"]: c for c in r["counters"]} for r in json.loads(capsys.readouterr().out)}
    assert abs(res["streamKernel"]["duration_us"]["change_pct"] + 20.0) < 1e-9 and abs(res["streamKernel"]["hbm_gbs"]["change_pct"] - 25.0) < 1e-9
    assert abs(res["mmaKernel"]["tensor_active_pct"]["other"] - 90.0) < 1e-9 and res["waitKernel"]["duration_us"]["change_pct"] == 0
    assert counters.main([str(tmp_path / "a.csv"), "--compare", str(tmp_path / "b.csv"), "--peaks", str(tmp_path / "p.json"), "--min-change", "5",
                          "--kernel-filter", "stream"]) == 0
    text = capsys.readouterr().out
    assert "== streamKernel" in text and "mmaKernel" not in text and "duration_us" in text and "dram_read_mb" not in text


def test_system_sampler_host_and_process_counters(tmp_path):
    """Without NVML the sampler still records the host (utilisation, frequency, load, memory) and, per watched process,
    resident set, CPU utilisation, threads, page faults and context switches."""
    import threading

    from rocm_systems_b200.tools import sysmon

    st = sysmon._proc_stat(os.getpid())
    assert st is not None and st["threads"] >= 1 and st["ticks"] >= 0 and st["minflt"] > 0
    stop = threading.Event()
    worker = threading.Thread(target=lambda: [sum(range(20000)) for _ in iter(lambda: stop.is_set(), True)])
    worker.start()
    with sysmon.SystemSampler(period_ms=30, pids=[os.getpid(), 2 ** 22 + 12345], gpu=False) as s:   # the second pid does not exist: skipped
        import time

        time.sleep(0.35)
    stop.set()
    worker.join()
    names = {n for n, _, _, _ in s.samples}
    assert {"host_cpu_util_percent", "host_mem_used_bytes", "host_load_1min", "process_rss_bytes", "process_threads", "process_cpu_util_percent",
            "process_page_faults_minor", "process_ctx_switches_voluntary"} <= names
    assert all(dev == os.getpid() for n, dev, _, _ in s.samples if n.startswith("process_"))
    threads = [v for n, _, _, v in s.samples if n == "process_threads"]
    assert max(threads) >= 2                                  # this thread and the worker at least
    assert all(v >= 0 for n, _, _, v in s.samples if n == "process_cpu_util_percent")
    assert s.write_csv(str(tmp_path / "s.csv")) == len(s.samples)


def test_a_run_ended_by_a_signal_keeps_its_ranges(tmp_path):
    """Markers under the launcher and the Python tracer: SIGTERM in mid-run still leaves the files, and the exit status says
    how the run ended; with --disable-signal-handlers the marker file is not written."""
    import signal
    import subprocess as sp

    child = ("import os, signal\nfrom rocm_systems_b200.utils import markers\nwith markers.range('before the end'):\n    pass\n"
             "os.kill(os.getpid(), signal.SIGTERM)\nimport time; time.sleep(5)\n")
    e = dict(os.environ, PYTHONPATH=str(ROOT))
    base = [sys.executable, "-m", "rocm_systems_b200.tools.prof", "--marker-trace", "-d"]
    p = sp.run([*base, str(tmp_path / "a"), "-o", "run", "--", sys.executable, "-c", child], env=e, capture_output=True, text=True, timeout=120)
    assert p.returncode == 128 + signal.SIGTERM, (p.returncode, p.stderr)
    assert "before the end" in (tmp_path / "a" / "run_regions.csv").read_text()
    p = sp.run([*base, str(tmp_path / "b"), "-o", "run", "--disable-signal-handlers", "--", sys.executable, "-c", child], env=e, capture_output=True, text=True, timeout=120)
    assert p.returncode == 128 + signal.SIGTERM and not (tmp_path / "b" / "run_regions.csv").exists()
    script = tmp_path / "s.py"
    script.write_text("import os, signal\ndef work():\n    return 1\nwork()\nos.kill(os.getpid(), signal.SIGTERM)\nimport time; time.sleep(5)\n")
    p = sp.run([sys.executable, "-m", "rocm_systems_b200.tools.pytrace", "-o", str(tmp_path / "py"), "-R", "^work$", "--", str(script)], env=e, capture_output=True,
               text=True, cwd=ROOT, timeout=120)
    assert p.returncode == 128 + signal.SIGTERM and "1 calls" in p.stderr
    assert '"work"' in next(tmp_path.glob("py.pytrace.*.csv")).read_text()
