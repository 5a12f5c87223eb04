"""The OpenMP tool (csrc/trace/ompt.cc): a stand-in for an OpenMP runtime loads ``libb200ompt.so`` the way
``OMP_TOOL_LIBRARIES`` is handled, offers ``ompt_set_callback`` and reports the events of a small program; regions must
come out as marker records with the right names, nesting, threads and pairing. The reference checks its OMPT support the
same way, through the callback records of an OpenMP target example (rocprofiler-sdk tests/openmp-tools)."""
import csv
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    from rocm_systems_b200.utils import build

    lib = build.build_ompt()
    if lib is None:
        pytest.skip("no OMPT header with this CUDA toolkit")
    assert build.build_lib().exists()
    exe = tmp_path_factory.mktemp("ompt") / "ompt_driver"
    subprocess.run(["g++", "-O1", "-std=c++17", "-I/usr/local/cuda/include", "-o", str(exe), str(ROOT / "tests" / "native" / "ompt_driver.cc"), "-ldl", "-lpthread"],
                   check=True)
    return exe, lib


def test_openmp_events_become_marker_records(driver, tmp_path):
    exe, lib = driver
    prefix = tmp_path / "om"
    env = dict(os.environ, B200COLL_TRACE="1", B200COLL_TRACE_FILE=str(prefix))
    r = subprocess.run([str(exe), str(lib)], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "callbacks 10" in r.stdout and "ompt driver done" in r.stdout, r.stdout + r.stderr   # masked was refused by the "runtime"
    with open(next(tmp_path.glob("om.markers.*.csv"))) as f:
        rows = list(csv.DictReader(f))
    names = [x["Function"] for x in rows]
    assert names.count("omp loop (500)") == 2 and "omp implicit task 0/2" in names and "omp implicit task 1/2" in names
    assert "omp implicit barrier" in names and names.count("omp thread end") == 2
    assert not any("1/1" in n for n in names)                                   # the initial task is not a region
    span = lambda x: (int(x["Start_Timestamp"]), int(x["End_Timestamp"]))  # noqa: E731
    by = {x["Function"]: x for x in rows}
    par = by["omp parallel (2 threads requested)"]
    tasks = [by["omp implicit task 0/2"], by["omp implicit task 1/2"]]
    assert tasks[0]["Thread_Id"] != tasks[1]["Thread_Id"]
    for t in tasks:
        assert span(par)[0] <= span(t)[0] and span(t)[1] <= span(par)[1]
    for x in rows:
        if x["Function"] == "omp loop (500)":
            task = next(t for t in tasks if t["Thread_Id"] == x["Thread_Id"])
            assert span(task)[0] <= span(x)[0] and span(x)[1] <= span(task)[1] and int(x["Depth"]) == int(task["Depth"]) + 1
    tgt = by["omp target (device 0, id 77)"]
    for inner in ("omp target data to device: 4096 B, device -1 -> 0 (id 77)", "omp target submit: 148 teams (id 77)"):
        assert span(tgt)[0] <= span(by[inner])[0] <= span(tgt)[1] and span(by[inner])[0] == span(by[inner])[1]
    assert "omp target enter data (device 1, id 78)" in by                      # closed when the tool was finalized


def test_tool_declines_without_the_marker_library_and_launcher_sets_it_up(driver, tmp_path):
    exe, lib = driver
    alone = tmp_path / "alone" / "libb200ompt.so"
    alone.parent.mkdir()
    alone.write_bytes(Path(lib).read_bytes())
    env = {k: v for k, v in os.environ.items() if k != "LD_LIBRARY_PATH"}
    r = subprocess.run([str(exe), str(alone)], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "tool declined" in r.stdout
    from rocm_systems_b200.tools import prof

    a = prof.parser().parse_args(["--openmp-trace", "--", "true"])
    e = prof.build_env(a, str(tmp_path / "t"))
    assert e["OMP_TOOL_LIBRARIES"].split(":")[0] == str(lib) and e["OMP_TOOL"] == "enabled"
    r = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.prof", "--openmp-trace", "--stats", "-d", str(tmp_path), "-o", "run", "--", str(exe), str(lib)],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0 and "omp parallel (2 threads requested)" in r.stdout, r.stdout + r.stderr
