"""The Kokkos Tools connector (csrc/trace/kokkosp.cc): a stand-in for the Kokkos runtime loads ``libb200kokkosp.so`` the
way ``KOKKOS_TOOLS_LIBS`` is loaded and issues the callbacks of a small program; every construct must come out as a marker
record with the right name, nesting and pairing, and the launcher must carry them into the trace database. The reference
tests its connector the same way, through a Kokkos example run under the tool and a check of the marker rows
(rocprofiler-sdk tests/kokkosp and the ``roctx`` rows its validation reads)."""
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

    lib = build.build_kokkosp()
    assert lib is not None and build.build_lib().exists()
    exe = tmp_path_factory.mktemp("kokkosp") / "kokkosp_driver"
    subprocess.run(["g++", "-O1", "-std=c++17", "-o", str(exe), str(ROOT / "tests" / "native" / "kokkosp_driver.cc"), "-ldl", "-lpthread"], check=True)
    return exe, lib


def _rows(prefix: Path) -> list:
    files = list(prefix.parent.glob(prefix.name + ".markers.*.csv"))
    assert len(files) == 1
    with open(files[0]) as f:
        return list(csv.DictReader(f))


def test_callbacks_become_marker_records(driver, tmp_path):
    exe, lib = driver
    prefix = tmp_path / "kk"
    env = dict(os.environ, B200COLL_TRACE="1", B200COLL_TRACE_FILE=str(prefix))
    r = subprocess.run([str(exe), str(lib)], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    ids = [int(x) for x in r.stdout.split()[1:]]
    assert len(set(ids)) == 4 and all(ids)                       # every begin callback handed back its own id
    rows = {row["Function"]: row for row in _rows(prefix)}
    assert set(rows) == {"parallel_reduce: dot", "parallel_for: axpy", "parallel_scan: prefix", "fence: Kokkos::fence after axpy",
                         "deep_copy: Host field_mirror <- Cuda field (4096 B)", "event: converged", "section: solver", "timestep", "section: left open"}
    span = lambda name: (int(rows[name]["Start_Timestamp"]), int(rows[name]["End_Timestamp"]))  # noqa: E731
    outer = span("timestep")
    for inner in ("parallel_for: axpy", "parallel_reduce: dot", "parallel_scan: prefix", "section: solver", "event: converged"):
        a, b = span(inner)
        assert outer[0] <= a <= b <= outer[1], inner
    # The reduce began inside the parallel_for and ended first; the parallel_for was ended from another thread.
    assert span("parallel_for: axpy")[0] <= span("parallel_reduce: dot")[0] and span("parallel_reduce: dot")[1] <= span("parallel_for: axpy")[1]
    assert span("event: converged")[0] == span("event: converged")[1] and rows["event: converged"]["Correlation_Id"] == "0"
    assert rows["deep_copy: Host field_mirror <- Cuda field (4096 B)"]["Depth"] == "1"    # pushed inside "timestep"
    assert span("section: left open")[1] >= span("section: left open")[0]                 # closed when the library was finalized


def test_memory_events_are_opt_in_and_markers_may_be_absent(driver, tmp_path):
    exe, lib = driver
    prefix = tmp_path / "mem"
    env = dict(os.environ, B200COLL_TRACE="1", B200COLL_TRACE_FILE=str(prefix), B200KOKKOSP_MEMORY_EVENTS="1")
    assert subprocess.run([str(exe), str(lib)], env=env, capture_output=True, timeout=120).returncode == 0
    names = [row["Function"] for row in _rows(prefix)]
    assert "allocate: Cuda field (4096 B)" in names and "deallocate: Cuda field (4096 B)" in names
    # A copy of the tool with no collective library beside it: every callback still returns.
    alone = tmp_path / "alone" / "libb200kokkosp.so"
    alone.parent.mkdir()
    alone.write_bytes(Path(lib).read_bytes())
    env = {k: v for k, v in os.environ.items() if k != "LD_LIBRARY_PATH"}
    r = subprocess.run([str(exe), str(alone)], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "not recorded" in r.stderr and r.stdout.startswith("ids 0 0 0 0")


def test_launcher_carries_kokkos_regions_into_the_database(driver, tmp_path):
    exe, lib = driver
    out = tmp_path / "run"
    r = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.prof", "--marker-trace", "--stats", "-d", str(tmp_path), "-o", "run", "--",
                        str(exe), str(lib)], capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "MARKER_API  parallel_for: axpy" in r.stdout and "9 records" in r.stderr, r.stdout + r.stderr
    import sqlite3

    db = sqlite3.connect(str(out) + ".db")
    tables = [t[0] for t in db.execute("select name from sqlite_master where type='table'")]
    found = sum(1 for t in tables for row in db.execute(f"select * from {t}") if any(isinstance(c, str) and c == "parallel_reduce: dot" for c in row))
    assert found >= 1
