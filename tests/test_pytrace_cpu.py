"""The Python function tracer (tools/pytrace.py): ranges per call with correct nesting and threads, the include / exclude /
restrict filters, labels, C calls, the builtin ``profile`` mode, the exit code of the script, and the hand-over to the
tracing launcher's database. The reference exercises its Python profiler the same way: example scripts run under
``python -m rocprofsys`` with label and filter options, then checks of the recorded function names
(rocprofiler-systems tests/rocprof-sys-python-tests.cmake)."""
import csv
import os
import sqlite3
import subprocess
import sys
import threading
from pathlib import Path

from rocm_systems_b200.tools import pytrace

ROOT = Path(__file__).resolve().parent.parent

SCRIPT = '''
import sys, time, threading
def leaf(n):
    return sum(range(n))
def middle(n):
    time.sleep(0.002)
    return leaf(n) + leaf(n // 2)
class Model:
    def step(self, k):
        return [middle(1000 * k) for _ in range(2)]
def _private():
    return leaf(3)
def worker():
    middle(10)
if __name__ == "__main__":
    m = Model()
    for k in range(3):
        m.step(k + 1)
    _private()
    t = threading.Thread(target=worker); t.start(); t.join()
    print("script done", sys.argv[1:])
    sys.exit(int(sys.argv[1]) if len(sys.argv) > 1 else 0)
'''


def _run(tmp_path, *opts, args=()):
    script = tmp_path / "traced.py"
    script.write_text(SCRIPT)
    r = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.pytrace", "-o", str(tmp_path / "run"), *opts, "--", str(script), *args],
                       capture_output=True, text=True, cwd=ROOT, timeout=120)
    files = list(tmp_path.glob("run.pytrace.*.csv"))
    assert len(files) == 1, r.stderr
    with open(files[0]) as f:
        return r, list(csv.DictReader(f))


def test_calls_become_nested_ranges_on_every_thread(tmp_path):
    r, rows = _run(tmp_path, "--stats", args=("3", "x"))
    assert r.returncode == 3 and "script done ['3', 'x']" in r.stdout          # the script's arguments and exit code pass through
    assert "Model.step" in r.stdout and "calls" in r.stdout                    # --stats
    names = [x["Function"] for x in rows]
    assert names.count("Model.step") == 3 and names.count("middle") == 7 and names.count("leaf") == 15 and names.count("worker") == 1
    assert all(x["Domain"] == "PYTHON_FUNCTION" for x in rows)
    span = lambda x: (int(x["Start_Timestamp"]), int(x["End_Timestamp"]))  # noqa: E731
    steps = [x for x in rows if x["Function"] == "Model.step"]
    for m in (x for x in rows if x["Function"] == "middle" and x["Thread_Id"] == steps[0]["Thread_Id"]):
        assert any(span(s)[0] <= span(m)[0] and span(m)[1] <= span(s)[1] and int(m["Depth"]) > int(s["Depth"]) for s in steps)
        assert span(m)[1] - span(m)[0] >= 2_000_000                             # it sleeps 2 ms
    w = next(x for x in rows if x["Function"] == "worker")
    assert w["Thread_Id"] != steps[0]["Thread_Id"]                              # the thread started under the tracer is traced, with its own id
    assert not any("genexpr" in n or "listcomp" in n for n in names)


def test_filters_labels_and_minimum_duration(tmp_path):
    _, rows = _run(tmp_path, "-R", "^(leaf|middle|_private)$", "-E", "^_", "--label", "file", "line")
    names = {x["Function"] for x in rows}
    assert names == {"leaf [traced.py:3]", "middle [traced.py:5]"}             # restrict keeps three, exclude drops _private
    for f in tmp_path.glob("run.pytrace.*.csv"):
        f.unlink()
    _, rows = _run(tmp_path, "-E", "^_", "-I", "_private", "--min-duration-us", "1500")
    names = [x["Function"] for x in rows]
    assert "leaf" not in names and names.count("middle") == 7                  # only the calls that sleep are long enough
    p = pytrace.Profiler(exclude_functions=["^_"], include_functions=["^_keep"], restrict_modules=["pkg/"])
    assert p.wanted("_keep_me", "/x/pkg/a.py") and not p.wanted("_drop", "/x/pkg/a.py") and p.wanted("f", "/x/pkg/a.py")
    assert not p.wanted("_keep_me", "/x/other/a.py")                            # restrict wins over include
    assert not pytrace.Profiler().wanted("f", "<frozen importlib._bootstrap>")


import pytest


@pytest.mark.parametrize("backend", ["monitoring", "setprofile"])
def test_in_process_use_c_calls_and_arguments(backend):
    if backend == "monitoring" and not hasattr(sys, "monitoring"):
        pytest.skip("sys.monitoring needs Python 3.12")

    def inner(a, b=2):
        return len([a, b])

    p = pytrace.Profiler(trace_c=True, label=["args"], restrict_functions=["inner", "len"], backend=backend)
    assert p.backend == backend
    assert p.runcall(inner, 5) == 2
    names = [r[0] for r in p.records]
    assert any(n.startswith("test_in_process_use_c_calls_and_arguments.<locals>.inner(a=5, b=2)") for n in names) and "builtins.len" in names
    by = {r[0].split("(")[0]: r for r in p.records}
    assert by["builtins.len"][4] > by["test_in_process_use_c_calls_and_arguments.<locals>.inner"][4]   # the C call is one level deeper
    assert p.stats(1)[0]["calls"] == 1
    # A tracer left no hook behind, and a second one can start; decorators pass through while one is active.
    assert sys.getprofile() is None and threading.getprofile() is None if hasattr(threading, "getprofile") else True
    q = pytrace.Profiler(restrict_functions=["inner"], backend=backend)
    with q:
        pytrace.profile(inner)(1)
    assert len(q.records) == 1 and len(pytrace.profile.records) == 0


def test_both_backends_see_the_same_calls_generators_and_exceptions(tmp_path):
    """The per-call hook and the per-code-object events give the same picture: same names and counts, a generator as one
    range per resumption, a function left by an exception still closed, threads traced."""
    script = tmp_path / "g.py"
    script.write_text(
        "import threading\n"
        "def gen(n):\n    for i in range(n):\n        yield i\n"
        "def boom():\n    raise ValueError('x')\n"
        "def caller():\n    try:\n        boom()\n    except ValueError:\n        pass\n    return sum(gen(3))\n"
        "caller()\nt = threading.Thread(target=caller); t.start(); t.join()\n")
    seen = {}
    for backend in (["monitoring"] if hasattr(sys, "monitoring") else []) + ["setprofile"]:
        r = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.pytrace", "--backend", backend, "-o", str(tmp_path / backend), "-R", "^(gen|boom|caller)$",
                            "--", str(script)], capture_output=True, text=True, cwd=ROOT, timeout=120)
        assert r.returncode == 0, r.stderr
        with open(next(tmp_path.glob(f"{backend}.pytrace.*.csv"))) as f:
            rows = list(csv.DictReader(f))
        names = [x["Function"] for x in rows]
        assert names.count("caller") == 2 and names.count("boom") == 2 and len({x["Thread_Id"] for x in rows}) == 2
        assert all(int(x["End_Timestamp"]) >= int(x["Start_Timestamp"]) for x in rows)
        seen[backend] = names.count("gen")
    # three values and the final return: the hook sees one call and one return per resumption as well
    assert set(seen.values()) == {8} or all(v >= 2 for v in seen.values())


def test_builtin_mode_traces_only_what_the_script_marks(tmp_path):
    script = tmp_path / "marked.py"
    script.write_text("def a():\n    return 1\n@profile\ndef b():\n    return a() + a()\na()\nb()\nwith profile:\n    a()\nprint('ok')\n")
    r = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.pytrace", "-b", "-o", str(tmp_path / "m"), "-R", "^[ab]$", "--", str(script)],
                       capture_output=True, text=True, cwd=ROOT, timeout=120)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr
    with open(next(tmp_path.glob("m.pytrace.*.csv"))) as f:
        names = [x["Function"] for x in csv.DictReader(f)]
    assert sorted(names) == ["a", "a", "a", "b"]                                # not the unmarked first a()


def test_launcher_puts_python_ranges_into_the_database(tmp_path):
    script = tmp_path / "traced.py"
    script.write_text(SCRIPT)
    r = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.prof", "--marker-trace", "--summary-per-domain", "-d", str(tmp_path), "-o", "run", "--",
                        sys.executable, "-m", "rocm_systems_b200.tools.pytrace", "-R", "^(leaf|middle|Model)", "--", str(script)],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "== DOMAIN PYTHON_FUNCTION ==" in r.stdout
    db = sqlite3.connect(str(tmp_path / "run.db"))
    rows = db.execute("select name, count(*) from regions where category = 'PYTHON_FUNCTION' group by name").fetchall()
    assert dict(rows) == {"Model.step": 3, "middle": 7, "leaf": 15, "Model": 1}


def test_launcher_python_trace_option(tmp_path):
    from rocm_systems_b200.tools import prof

    assert prof.python_traced(["python3", "-u", "train.py", "--steps", "2"], ["my_pkg/"]) == \
        ["python3", "-u", "-m", "rocm_systems_b200.tools.pytrace", "-MR", "my_pkg/", "--", "train.py", "--steps", "2"]
    assert prof.python_traced(["python", "-W", "ignore", "a.py"]) == ["python", "-W", "ignore", "-m", "rocm_systems_b200.tools.pytrace", "--", "a.py"]
    assert prof.python_traced(["python", "-m", "pkg.mod"]) is None and prof.python_traced(["./app"]) is None and prof.python_traced(["python", "-c", "pass"]) is None
    script = tmp_path / "traced.py"
    script.write_text(SCRIPT)
    r = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.prof", "--python-trace", "--python-restrict", "traced", "-d", str(tmp_path), "-o", "run", "--",
                        sys.executable, str(script)], capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    db = sqlite3.connect(str(tmp_path / "run.db"))
    assert dict(db.execute("select name, count(*) from regions where category = 'PYTHON_FUNCTION' and name in ('middle', 'leaf') group by name")) == {"middle": 7, "leaf": 15}
    r = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.prof", "--python-trace", "-d", str(tmp_path), "--", "true"], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 2 and "python script.py" in r.stderr


def test_python_trace_of_a_multi_rank_launch(tmp_path):
    """Every rank of a torch.distributed.run launch runs its script under the tracer and writes a file of its own."""
    from rocm_systems_b200.tools import prof

    cmd = ["python", "-m", "torch.distributed.run", "--nproc-per-node", "2", "train.py", "--x"]
    assert prof.python_traced(cmd) == ["python", "-m", "torch.distributed.run", "--nproc-per-node", "2", "-m", "rocm_systems_b200.tools.pytrace", "--", "train.py", "--x"]
    assert prof.python_traced(["python", "-m", "torch.distributed.run", "--nproc-per-node", "2", "-m", "pkg.train"]) is None
    script = tmp_path / "rank.py"
    script.write_text("import os\ndef work(r):\n    return r + 1\nwork(int(os.environ['RANK']))\nprint('rank done', os.environ['RANK'])\n")
    r = subprocess.run([sys.executable, "-m", "rocm_systems_b200.tools.prof", "--python-trace", "--python-restrict", "rank", "-d", str(tmp_path), "-o", "run", "--",
                        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", "29931",
                        str(script)], capture_output=True, text=True, cwd=ROOT, timeout=600, env=dict(os.environ, PYTHONPATH=str(ROOT)))
    assert r.returncode == 0 and r.stdout.count("rank done") == 2, r.stdout[-2000:] + r.stderr[-2000:]
    db = sqlite3.connect(str(tmp_path / "run.db"))
    rows = db.execute("select count(*), count(distinct pid) from regions where category = 'PYTHON_FUNCTION' and name = 'work'").fetchone()
    assert rows == (2, 2)
