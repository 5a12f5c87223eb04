"""The causal profiler (csrc/prof/causal.cc, tools/causal.py) on a native program whose answer is known: every iteration
runs ``cpu_slow_func`` and ``cpu_fast_func`` side by side and waits for both, the fast one doing 80 % of the slow one's
work. Making the slow one 20 % faster must speed the program up by about 20 %, 30 % faster by no more (the fast one is
the bound then), and making the fast one faster by nothing. This is the reference's own end-to-end validation
(rocprofiler-systems tests/rocprof-sys-causal-tests.cmake: slow-func 10/20/30 -> 10/20/20, fast-func -> 0/0/0, checked by
tests/validate-causal-json.py), on both ways the target hands work to its threads: threads created and joined per
iteration, and a pool woken through a mutex and condition variables."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

from rocm_systems_b200.tools import causal

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "rocm_systems_b200" / "lib" / "libb200causal.so"


@pytest.fixture(scope="module")
def target(tmp_path_factory):
    from rocm_systems_b200.utils import build

    assert build.build_causal() == LIB
    exe = tmp_path_factory.mktemp("causal") / "causal_target"
    subprocess.run(["g++", "-O1", "-g", "-std=c++17", f"-I{ROOT / 'rocm_systems_b200' / 'csrc' / 'include'}", "-o", str(exe),
                    str(ROOT / "tests" / "native" / "causal_target.cc"), "-lpthread", "-ldl"], check=True)
    return exe


TEXT = "\n".join([
    "startup\ttime=1",
    "experiment\tselected=f\tspeedup=0.00\tduration=1000\tselected-samples=5\treal-duration=1000\tpaused=0",
    "throughput-point\tname=it\tdelta=10",
    "latency-point\tname=item\tarrivals=10\tdepartures=10\tdifference=0",
    "experiment\tselected=f\tspeedup=0.00\tduration=1100\tselected-samples=5",
    "throughput-point\tname=it\tdelta=10",
    "experiment\tselected=f\tspeedup=0.50\tduration=800\tselected-samples=5\treal-duration=1200\tpaused=400",
    "throughput-point\tname=it\tdelta=10",
    "experiment\tselected=g\tspeedup=0.50\tduration=800\tselected-samples=5",     # no baseline for g: not reported
    "throughput-point\tname=it\tdelta=10",
    "runtime\ttime=99\tsamples=20",
    "throughput-point\tname=stray\tdelta=1",                                       # outside an experiment: ignored
])


def test_parse_and_predictions():
    ex = causal.parse(TEXT)
    assert len(ex) == 4 and ex[2]["speedup"] == 50 and ex[2]["real_duration"] == 1200 and ex[1]["real_duration"] == 1100
    assert ex[0]["latency"]["item"]["departures"] == 10 and "stray" not in ex[3]["throughput"]
    res = causal.analyze(ex)
    by = {(r["selected"], r["point"], r["kind"]): r for r in res}
    assert set(by) == {("f", "it", "throughput"), ("f", "item", "latency")}
    r = by[("f", "it", "throughput")]
    assert r["baseline_period_ns"] == pytest.approx(105.0)
    rows = {row["speedup"]: row for row in r["rows"]}
    assert rows[0]["program_speedup"] == pytest.approx(0.0) and rows[0]["experiments"] == 2
    assert rows[50]["program_speedup"] == pytest.approx(100 * (1 - 80 / 105))
    assert r["impact"] == pytest.approx(0.5 * rows[50]["program_speedup"])            # area under the curve per unit of speed-up
    assert causal.analyze(ex, point="nope") == []
    assert causal.analyze(ex, min_experiments=2)[0]["rows"][-1]["speedup"] == 0      # the single run at 50 % is dropped
    assert "f  [throughput point: it]" in causal.format_report(res)
    assert causal.validate(res, [("f", "it", 50, 24.0, 2.0)]) == []
    assert len(causal.validate(res, [("f", "it", 50, 60.0, 2.0), ("f", "it", 70, 0.0, 2.0)])) == 2


def test_latency_point_by_littles_law():
    """Items in flight at the ends of the experiments turn a latency point into the time an item spends in flight:
    sum(in flight x duration) / sum(arrivals); with nothing in flight the time per departure is compared instead."""
    text = "\n".join([
        "experiment\tselected=f\tspeedup=0.00\tduration=1000\tselected-samples=5",
        "latency-point\tname=q\tarrivals=10\tdepartures=10\tdifference=4",
        "experiment\tselected=f\tspeedup=0.00\tduration=3000\tselected-samples=5",
        "latency-point\tname=q\tarrivals=30\tdepartures=28\tdifference=6",
        "experiment\tselected=f\tspeedup=0.50\tduration=1000\tselected-samples=5",
        "latency-point\tname=q\tarrivals=20\tdepartures=20\tdifference=4",
    ])
    r = causal.analyze(causal.parse(text))[0]
    assert r["kind"] == "latency (time in flight)"
    assert r["baseline_period_ns"] == pytest.approx((4 * 1000 + 6 * 3000) / 40)          # 550 ns in flight per item
    rows = {row["speedup"]: row["program_speedup"] for row in r["rows"]}
    assert rows[50] == pytest.approx(100 * (1 - (4 * 1000 / 20) / 550))
    plain = causal.analyze(causal.parse(text.replace("difference=4", "difference=0").replace("difference=6", "difference=0")))[0]
    assert plain["kind"] == "latency" and plain["baseline_period_ns"] == pytest.approx(4000 / 38)


def test_end_to_end_plan_and_environment(tmp_path):
    ap_args = ["run", "-o", str(tmp_path / "x.coz"), "-e", "-n", "2", "-s", "0", "20", "-F", "^a$", "^b$", "--", "prog"]
    import argparse  # noqa: F401

    captured = {}
    real_run = causal.cmd_run
    try:
        causal.cmd_run = lambda a: captured.setdefault("a", a) and 0
        causal.main(ap_args)
    finally:
        causal.cmd_run = real_run
    a = captured["a"]
    jobs = causal.plan(a)
    assert len(jobs) == 2 * 2 * 2 and {j["function"] for j in jobs} == {"^a$", "^b$"} and {j["speedup"] for j in jobs} == {0, 20}
    env = causal.environment(a, 20, "^a$")
    assert env["B200CAUSAL_END_TO_END"] == "1" and env["B200CAUSAL_FIXED_SPEEDUP"] == "20" and env["B200CAUSAL_FUNCTION_SCOPE"] == "^a$"
    assert env["LD_PRELOAD"].split(":")[0] == str(LIB) and env["B200CAUSAL_FILE"].endswith("x.coz")
    a.end_to_end = False
    assert causal.plan(a) == [{"speedup": None, "function": None, "source": None}] * 2


def _spread_ok(results, of_the_mean=False):
    """A loaded machine shows as a wide spread of the baseline; then the numbers mean nothing either way. With many short
    experiments the spread of one experiment is mostly the +/- 1 visit at its edges, which averages out in the prediction:
    there the spread of the mean (stddev / sqrt(experiments)) is what has to be small."""
    def spread(r):
        n = next((row["experiments"] for row in r["rows"] if row["speedup"] == 0), 1)
        return r["baseline_stddev"] / (n ** 0.5 if of_the_mean else 1.0)
    return all(spread(r) < (3.0 if of_the_mean else 6.0) for r in results)


def test_end_to_end_predictions_match_the_known_answer(target, tmp_path):
    out = tmp_path / "e2e.coz"
    rc = causal.main(["run", "-o", str(out), "-e", "-n", "2", "-s", "0", "20", "30", "-F", "^cpu_slow_func$", "^cpu_fast_func$", "--",
                      str(target), "24", "80", "4000000", "spawn"])
    assert rc == 0
    ex = causal.parse(out.read_text())
    assert len(ex) == 12 and {e["selected"] for e in ex} == {"cpu_slow_func", "cpu_fast_func"}
    assert all(e["throughput"]["iteration"] == 24 and e["latency"]["item"]["departures"] == 24 for e in ex)
    assert all(e["selected_samples"] > 20 for e in ex)
    assert all((e["real_duration"] > e["duration"]) == (e["speedup"] > 0) for e in ex)   # pauses only when something is sped up
    res = causal.analyze(ex, point="iteration")
    if not _spread_ok(res):
        pytest.skip("baseline runs differ by more than 6 %: the machine is busy")
    bad = causal.validate(res, [("cpu_slow_func", "iteration", 20, 20.0, 7.0), ("cpu_slow_func", "iteration", 30, 20.0, 8.0),
                                ("cpu_fast_func", "iteration", 20, 0.0, 7.0), ("cpu_fast_func", "iteration", 30, 0.0, 7.0)])
    assert bad == [], causal.format_report(res)
    # The report command on the same file, with the checks as arguments.
    r = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.causal", "report", str(out), "--point", "iteration", "--validate",
                        "cpu_slow_func", "iteration", "20", "20", "9"], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0 and "cpu_slow_func  [throughput point: iteration]" in r.stdout, r.stdout + r.stderr


LINE_TABLE = """Contents of the .debug_line section:

CU: src/solver.cc:
File name                            Line number    Starting address    View    Stmt
solver.cc                                     10              0x1000               x
solver.cc                                     11              0x1008               x
solver.cc                                     11              0x1008       1
solver.cc                                     10              0x1010
solver.cc                                     12              0x1018               x

/usr/include/c++/13/cmath:
cmath                                        100              0x1020               x
cmath                                          -              0x1030

src/solver.cc:
solver.cc                                     11              0x2000               x
solver.cc                                      -              0x2004
"""


def test_line_table_rows_become_ranges_per_line(monkeypatch, tmp_path):
    rows = causal.decode_line_table(LINE_TABLE)
    assert rows == [("src/solver.cc", 10, 0x1000, 0x1008), ("src/solver.cc", 11, 0x1008, 0x1010), ("src/solver.cc", 10, 0x1010, 0x1018),
                    ("src/solver.cc", 12, 0x1018, 0x1020), ("/usr/include/c++/13/cmath", 100, 0x1020, 0x1030), ("src/solver.cc", 11, 0x2000, 0x2004)]
    monkeypatch.setattr(causal.subprocess, "run", lambda *a, **k: type("R", (), {"returncode": 0, "stdout": LINE_TABLE, "stderr": ""})())
    assert causal.source_ranges("exe", [r"solver\.cc:11$"]) == {"solver.cc:11": [(0x1008, 0x1010), (0x2000, 0x2004)]}
    every = causal.source_ranges("exe", [r"solver\.cc"])
    assert set(every) == {"solver.cc:10", "solver.cc:11", "solver.cc:12"} and every["solver.cc:10"] == [(0x1000, 0x1008), (0x1010, 0x1018)]
    assert causal.source_ranges("exe", ["nothing"]) == {}
    causal.write_source_ranges(tmp_path / "r", every)
    assert (tmp_path / "r").read_text().splitlines()[1] == "solver.cc:11\t1008-1010,2000-2004"


def test_source_line_scope_matches_the_known_answer(target, tmp_path):
    src = (ROOT / "tests" / "native" / "causal_target.cc").read_text().splitlines()
    slow = next(i for i, l in enumerate(src, 1) if "SLOW_LINE" in l and "for (" in l)
    fast = next(i for i, l in enumerate(src, 1) if "FAST_LINE" in l and "for (" in l)
    out = tmp_path / "lines.coz"
    rc = causal.main(["run", "-o", str(out), "-e", "-n", "2", "-s", "0", "20", "-S", rf"causal_target\.cc:{slow}$", rf"causal_target\.cc:{fast}$", "--",
                      str(target), "24", "80", "4000000", "spawn"])
    assert rc == 0
    ex = causal.parse(out.read_text())
    assert {e["selected"] for e in ex} == {f"causal_target.cc:{slow}", f"causal_target.cc:{fast}"} and len(ex) == 8
    assert all(e["selected_samples"] > 20 for e in ex)
    res = causal.analyze(ex, point="iteration")
    if not _spread_ok(res):
        pytest.skip("baseline runs differ by more than 6 %: the machine is busy")
    bad = causal.validate(res, [(f"causal_target.cc:{slow}", "iteration", 20, 20.0, 7.0), (f"causal_target.cc:{fast}", "iteration", 20, 0.0, 7.0)])
    assert bad == [], causal.format_report(res)


@pytest.mark.parametrize("backend,announcement", [("perf", "per-thread CPU-clock events"), ("timer", "process CPU-time timer")])
def test_both_sample_sources(target, tmp_path, backend, announcement):
    """The per-thread CPU-clock events give samples at the rate asked for, the process timer one per scheduler tick; both
    predict the known answer. Where the kernel refuses perf_event_open the perf case is skipped (auto then uses the timer)."""
    out = tmp_path / f"{backend}.coz"
    for speedup in (0, 20, 0, 20):
        env = dict(os.environ, LD_PRELOAD=str(LIB), B200CAUSAL_FILE=str(out), B200CAUSAL_BACKEND=backend, B200CAUSAL_END_TO_END="1",
                   B200CAUSAL_FUNCTION_SCOPE="^cpu_slow_func$", B200CAUSAL_FIXED_SPEEDUP=str(speedup), B200CAUSAL_VERBOSE="1", B200CAUSAL_FREQ="1000")
        r = subprocess.run([str(target), "24", "80", "4000000", "spawn"], env=env, capture_output=True, text=True, timeout=300)
        if backend == "perf" and "not available here" in r.stderr:
            pytest.skip("perf_event_open is not allowed on this machine")
        assert r.returncode == 0 and announcement in r.stderr, r.stderr
    ex = causal.parse(out.read_text())
    assert len(ex) == 4
    per_second = ex[0]["selected_samples"] / (ex[0]["real_duration"] / 1e9)
    assert per_second > (250 if backend == "perf" else 20), per_second     # 1 kHz of CPU time asked for (less per wall second on a busy machine); the timer gives one sample per scheduler tick
    res = causal.analyze(ex, point="iteration")
    if not _spread_ok(res):
        pytest.skip("baseline runs differ by more than 6 %: the machine is busy")
    assert causal.validate(res, [("cpu_slow_func", "iteration", 20, 20.0, 7.0)]) == [], causal.format_report(res)


def test_experiments_drawn_while_a_thread_pool_runs(target, tmp_path):
    out = tmp_path / "pool.coz"
    env = dict(os.environ, LD_PRELOAD=str(LIB), B200CAUSAL_FILE=str(out), B200CAUSAL_FIXED_SPEEDUP="0,20", B200CAUSAL_EXPERIMENT_SECONDS="0.4",
               B200CAUSAL_RANDOM_SEED="11", B200CAUSAL_VERBOSE="1", B200CAUSAL_FUNCTION_SCOPE="^cpu_(slow|fast)_func$")
    r = subprocess.run([str(target), "600", "80", "2000000", "pool"], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "done 600" in r.stdout
    assert "Starting causal experiment #1" in r.stderr
    text = out.read_text()
    assert text.startswith("startup\ttime=") and text.rstrip().splitlines()[-1].startswith("runtime\ttime=")
    ex = causal.parse(text)
    assert len(ex) >= 8
    assert {e["selected"] for e in ex} == {"cpu_slow_func", "cpu_fast_func"}
    assert {e["speedup"] for e in ex} == {0, 20}
    res = [x for x in causal.analyze(ex, point="iteration") if x["selected"] in ("cpu_slow_func", "cpu_fast_func")]
    if len(res) < 2 or not _spread_ok(res, of_the_mean=True) or any(len(x["rows"]) < 2 for x in res) or \
            any(row["experiments"] < 2 for x in res for row in x["rows"]):
        pytest.skip("not both functions drawn at least twice at both speed-ups (an experiment sees a whole number of visits: one is too noisy), or a busy machine")
    by = {x["selected"]: {row["speedup"]: row["program_speedup"] for row in x["rows"]} for x in res}
    assert by["cpu_slow_func"][20] > by["cpu_fast_func"][20] + 3.0, causal.format_report(res)
    assert 8.0 < by["cpu_slow_func"][20] < 32.0 and abs(by["cpu_fast_func"][20]) < 12.0, causal.format_report(res)


def test_pipeline_example_under_the_profiler(tmp_path):
    """The example of the examples folder: experiments select the stage functions (callers of the sampled code are
    candidates), both kinds of progress point are recorded, and the middle stage is the one whose speed-up pays."""
    exe = tmp_path / "causal_pipeline"
    subprocess.run(["g++", "-O1", "-g", "-std=c++17", f"-I{ROOT / 'rocm_systems_b200' / 'csrc' / 'include'}", "-o", str(exe),
                    str(ROOT / "examples" / "causal_pipeline.cc"), "-lpthread", "-ldl"], check=True)
    out = tmp_path / "p.coz"
    rc = causal.main(["run", "-o", str(out), "-s", "0", "40", "--experiment-seconds", "0.3", "--seed", "5", "-F", "^(decode|transform|write_out)$", "--",
                      str(exe), "7000"])
    assert rc == 0
    ex = causal.parse(out.read_text())
    assert len(ex) >= 8 and {e["selected"] for e in ex} <= {"decode", "transform", "write_out"}
    assert all("item" in e["throughput"] and "in flight" in e["latency"] for e in ex)
    res = {r["selected"]: r for r in causal.analyze(ex, point="item")}
    if "transform" not in res or len(res["transform"]["rows"]) < 2 or not _spread_ok(list(res.values())):
        pytest.skip("the middle stage was not drawn at both speed-ups, or a busy machine")
    at40 = {row["speedup"]: row["program_speedup"] for row in res["transform"]["rows"]}[40]
    assert 22.0 < at40 < 50.0, causal.format_report(list(res.values()))


def test_without_the_library_the_marks_do_nothing(target):
    r = subprocess.run([str(target), "2", "80", "100000"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "done 2" in r.stdout
    from rocm_systems_b200.utils import causal as marks

    marks.progress("x")
    with marks.item("y"):
        pass
    assert marks.active() is False
