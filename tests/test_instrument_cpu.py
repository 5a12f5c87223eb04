"""Function instrumentation (csrc/prof/instrument.cc, tools/instrument.py) on a program with a known call tree, built with
the flags the tool prints: call counts, inclusive against exclusive time, the thread's calls, marker ranges for long
calls only, and the coverage figure with the one cold function named. The reference validates its instrumentation modes
the same way: an example is instrumented, run, and the output is checked for the expected functions and for the coverage
numbers (rocprofiler-systems tests/rocprof-sys-instrument-tests.cmake, tests/rocprof-sys-code-coverage-tests.cmake)."""
import csv
import json
import subprocess
import sys
from pathlib import Path

import pytest

from rocm_systems_b200.tools import instrument

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def target(tmp_path_factory):
    exe = tmp_path_factory.mktemp("instr") / "instrument_target"
    subprocess.run(["g++", "-O1", "-g", "-std=c++17", *instrument.FLAGS.split(), "-o", str(exe), str(ROOT / "tests" / "native" / "instrument_target.cc"), "-lpthread"],
                   check=True)
    return exe


def test_statistics_ranges_and_coverage(target, tmp_path):
    prefix = tmp_path / "run"
    rc = instrument.main(["run", "-o", str(prefix), "--trace", "--min-us", "1500", "--", str(target)])
    assert rc == 0
    doc = instrument.merge(str(prefix))
    by = {r["function"]: r for r in doc["functions"]}
    assert doc["processes"] == 1 and set(by) == {"main", "app::Solver::run(int)", "outer()", "inner(int)", "main::{lambda()#1}::operator()() const"}
    assert by["inner(int)"]["calls"] == 7 and by["outer()"]["calls"] == 3 and by["app::Solver::run(int)"]["calls"] == 3 and by["main"]["calls"] == 1
    assert by["inner(int)"]["inclusive_ns"] == by["inner(int)"]["exclusive_ns"] >= 7 * 1_000_000           # a leaf; it sleeps 1 ms
    o = by["outer()"]
    assert o["inclusive_ns"] >= 3 * 4_000_000 and 3 * 2_000_000 <= o["exclusive_ns"] < o["inclusive_ns"] - 5_000_000
    r = by["app::Solver::run(int)"]
    assert r["inclusive_ns"] >= 12_000_000 and r["exclusive_ns"] < r["inclusive_ns"] / 2      # nearly all of its time is in outer()
    assert doc["functions"][0]["function"] == "main"                                                       # sorted by inclusive time
    c = doc["coverage"]
    assert c["functions_defined"] == 6 and c["functions_called"] == 5 and c["uncalled"] == ["never_called()"] and c["percent"] == pytest.approx(83.33)
    with open(next(tmp_path.glob("run.markers.*.csv"))) as f:
        names = [r["Function"] for r in csv.DictReader(f)]
    assert names.count("outer()") == 3 and names.count("main") == 1 and "inner(int)" not in names            # 1 ms calls are under the threshold
    r = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.instrument", "report", str(prefix), "--coverage"], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0 and "5 of 6 functions called (83.33 %)" in r.stdout and "never called: never_called()" in r.stdout and "outer()" in r.stdout


def test_without_tracing_and_over_two_processes(target, tmp_path):
    prefix = tmp_path / "two"
    assert instrument.main(["run", "-o", str(prefix), "--", str(target)]) == 0
    assert instrument.main(["run", "-o", str(prefix), "--", str(target), "a", "b", "c", "d", "e"]) == 0       # this one calls never_called()
    assert not list(tmp_path.glob("two.markers.*.csv"))                                                      # no marker library without --trace
    doc = instrument.merge(str(prefix))
    assert doc["processes"] == 2 and doc["coverage"]["functions_called"] == 6 and doc["coverage"]["uncalled"] == []
    assert {r["function"]: r["calls"] for r in doc["functions"]}["inner(int)"] == 14
    assert json.loads(subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.instrument", "report", str(prefix), "--json"], capture_output=True, text=True,
                                     cwd=ROOT).stdout)["coverage"]["percent"] == 100.0
    assert "-finstrument-functions" in subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.instrument", "flags"], capture_output=True, text=True,
                                                      cwd=ROOT).stdout


def test_an_uninstrumented_program_is_left_alone(tmp_path):
    prefix = tmp_path / "plain"
    assert instrument.main(["run", "-o", str(prefix), "--", "true"]) == 0
    doc = instrument.merge(str(prefix))
    assert doc["functions"] == [] and doc["processes"] == 1
