"""The host call-stack sampler (csrc/prof/sampler.cc) on a small native program with a known profile: one thread burns
CPU in ``burn_cycles``, another sleeps in ``idle_wait``. CPU-time sampling must see only the burner, wall-clock sampling
both; the tracing launcher must carry the samples into the database, the statistics, the folded stacks and the Perfetto
export. Mirrors how the reference validates its sampling mode: run an example under the sampler, then check the output
for the expected call-stack entries (rocprofiler-systems tests/rocprof-sys-testing.cmake, the ``sampling`` runs)."""
import ctypes
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "rocm_systems_b200" / "lib" / "libb200sample.so"


@pytest.fixture(scope="module")
def target(tmp_path_factory):
    from rocm_systems_b200.utils import build

    assert build.build_sampler() == LIB
    exe = tmp_path_factory.mktemp("sampler") / "target"
    subprocess.run(["g++", "-O1", "-rdynamic", "-o", str(exe), str(ROOT / "tests" / "native" / "sampler_target.cc"), "-lpthread"], check=True)
    return exe


def _folded(path: Path) -> dict:
    out = {}
    for line in path.read_text().splitlines():
        stack, _, n = line.rpartition(" ")
        out[stack] = int(n)
    return out


def _run(target, tmp_path, clock: str) -> tuple:
    prefix = tmp_path / f"s_{clock}"
    env = dict(os.environ, LD_PRELOAD=str(LIB), B200SAMPLE_PREFIX=str(prefix), B200SAMPLE_CLOCK=clock, B200SAMPLE_FREQ="200")
    subprocess.run([str(target)], env=env, check=True, capture_output=True, timeout=120)
    folded = list(tmp_path.glob(f"s_{clock}.*.folded"))
    csvs = list(tmp_path.glob(f"s_{clock}.*.samples.csv"))
    assert len(folded) == 1 and len(csvs) == 1
    return _folded(folded[0]), csvs[0].read_text().splitlines()


def test_cpu_clock_sees_the_thread_that_burns(target, tmp_path):
    stacks, rows = _run(target, tmp_path, "cpu")
    total = sum(stacks.values())
    assert total >= 50 and len(rows) == total + 1 and rows[0] == "timestamp_ns,tid,depth,clock,stack"
    burning = sum(n for s, n in stacks.items() if s.endswith("burn_cycles"))
    assert burning >= 0.8 * total
    assert all("main" in s for s in stacks if s.endswith("burn_cycles"))         # outer frames come first
    assert not any("idle_wait" in s for s in stacks)                             # a sleeping thread uses no CPU time
    ts = [int(r.split(",")[0]) for r in rows[1:]]
    assert ts == sorted(ts) or len(set(r.split(",")[1] for r in rows[1:])) > 1  # one thread: time-ordered


def test_wall_clock_sees_blocked_threads_too(target, tmp_path):
    stacks, rows = _run(target, tmp_path, "wall")
    total = sum(stacks.values())
    idle = sum(n for s, n in stacks.items() if "idle_wait" in s)
    burning = sum(n for s, n in stacks.items() if s.endswith("burn_cycles"))
    assert idle >= 0.25 * total and burning >= 0.25 * total
    assert len({r.split(",")[1] for r in rows[1:]}) >= 2                         # samples carry the thread they were taken on
    assert all(r.split(",")[3] == "wall" for r in rows[1:])


def test_launcher_imports_samples_and_reports_them(target, tmp_path):
    from rocm_systems_b200.tools import prof, tracedb

    out = tmp_path / "out"
    rc = prof.main(["--host-sampling", "--sampling-freq", "200", "--output-format", "db", "pftrace", "-d", str(out), "--", str(target)])
    assert rc == 0
    with tracedb.TraceDB(str(out / "trace.db")) as db:
        n = db.query("select count(*) from host_sample")[1][0][0]
        prof_rows = db.host_profile(5)
        s = db.summary()
    assert n >= 50 and prof_rows[0]["function"] == "burn_cycles" and prof_rows[0]["self_pct"] >= 80.0
    main_row = next(r for r in s["host_samples"] if r["function"] == "main")
    assert main_row["self"] == 0 or main_row["self_pct"] < 20.0
    assert main_row["inclusive_pct"] >= 80.0
    folded = _folded(out / "trace.folded")
    assert sum(folded.values()) == n and not list(out.glob("trace.*.folded"))
    events = json.loads((out / "trace.perfetto.json").read_text())["traceEvents"]
    inst = [e for e in events if e.get("cat") == "host_sample"]
    assert len(inst) == n and inst[0]["ph"] == "i" and inst[0]["args"]["stack"][-1] == inst[0]["name"]


def test_in_process_api_rejects_bad_arguments_and_round_trips(tmp_path):
    code = f"""
import ctypes, sys
lib = ctypes.CDLL({str(LIB)!r})
lib.b200sampleStart.argtypes = [ctypes.c_double, ctypes.c_int]
lib.b200sampleCount.restype = ctypes.c_uint64
assert lib.b200sampleStart(0.0, 0) == -2 and lib.b200sampleStart(100.0, 7) == -2
assert lib.b200sampleStart(500.0, 0) == 0 and lib.b200sampleStart(500.0, 0) == -1
x = 0
for i in range(4000000): x += i * i
assert lib.b200sampleWrite({str(tmp_path / 'early')!r}.encode()) == -1          # not while running
assert lib.b200sampleStop() == 0 and lib.b200sampleStop() == 0
n = lib.b200sampleCount()
assert n > 5, n
assert lib.b200sampleWrite({str(tmp_path / 'inproc')!r}.encode()) == 2
lib.b200sampleClear()
assert lib.b200sampleCount() == 0
print(n)
"""
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr
    rows = (tmp_path / "inproc.samples.csv").read_text().splitlines()
    assert len(rows) == int(p.stdout.strip()) + 1
    assert any("_PyEval_EvalFrameDefault" in r for r in rows)


def test_python_context_manager():
    code = """
from rocm_systems_b200.utils.profiler import HostSampler
import zlib
with HostSampler(freq_hz=500, clock="cpu") as s:
    data = bytes(range(256)) * 40000
    for _ in range(12): zlib.compress(data, 6)
assert s.count() > 5 and s.dropped() == 0
top = s.top(3)
print(top)
assert any("deflate" in fn or "longest_match" in fn or "compress" in fn or "libz" in fn for fn, _ in top), top
assert abs(sum(share for _, share in s.top(10000)) - 1.0) < 1e-9
"""
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, env=dict(os.environ, PYTHONPATH=str(ROOT)))
    assert p.returncode == 0, p.stdout + p.stderr


def test_samples_survive_a_terminating_signal(target, tmp_path):
    import signal
    import time

    prefix = tmp_path / "killed"
    env = dict(os.environ, LD_PRELOAD=str(LIB), B200SAMPLE_PREFIX=str(prefix), B200SAMPLE_FREQ="200", B200SAMPLE_SIGNALS="1")
    p = subprocess.Popen([str(target)], env=env, stdout=subprocess.DEVNULL)
    time.sleep(0.5)
    p.send_signal(signal.SIGTERM)
    assert p.wait(timeout=30) == -signal.SIGTERM                        # the signal still ends the program
    stacks = _folded(next(tmp_path.glob("killed.*.folded")))
    assert sum(stacks.values()) >= 5 and any(s.endswith("burn_cycles") for s in stacks)
    env.pop("B200SAMPLE_SIGNALS")
    env["B200SAMPLE_PREFIX"] = str(tmp_path / "lost")
    p = subprocess.Popen([str(target)], env=env, stdout=subprocess.DEVNULL)
    time.sleep(0.3)
    p.send_signal(signal.SIGTERM)
    assert p.wait(timeout=30) == -signal.SIGTERM and not list(tmp_path.glob("lost.*"))


def test_sampling_window(target, tmp_path):
    """B200SAMPLE_DURATION: samples are taken for that long, the program runs on, the files are written at its end."""
    prefix = tmp_path / "win"
    env = dict(os.environ, LD_PRELOAD=str(LIB), B200SAMPLE_PREFIX=str(prefix), B200SAMPLE_CLOCK="wall", B200SAMPLE_FREQ="100", B200SAMPLE_DURATION="0.3")
    subprocess.run([str(target)], env=env, check=True, capture_output=True, timeout=120)
    rows = next(tmp_path.glob("win.*.samples.csv")).read_text().splitlines()[1:]
    ts = [int(r.split(",")[0]) for r in rows]
    assert len(ts) >= 10 and (max(ts) - min(ts)) / 1e9 < 0.6          # the target runs for about a second
