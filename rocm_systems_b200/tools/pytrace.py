"""Python function tracing: every call of a Python function (optionally of C functions too) becomes a range on the clock of
the other tracers, so that the interpreter's side of a training step lines up with kernels, copies and collectives.

    python -m rocm_systems_b200.tools.pytrace -o out/run --stats -- train.py --steps 4
    python -m rocm_systems_b200.tools.pytrace -MR 'rocm_systems_b200/' -E '^_' --min-duration-us 50 -- train.py
    python -m rocm_systems_b200.tools.prof --kernel-trace --marker-trace -d out -o run -- \\
        python -m rocm_systems_b200.tools.pytrace -- train.py          # one database with both (the prefix is inherited)

In a program::

    from rocm_systems_b200.tools.pytrace import Profiler, profile
    with Profiler(restrict_modules=["my_pkg/"]) as p: step()
    @profile
    def hot(): ...

The ranges are written as ``<prefix>.pytrace.<pid>.csv`` (domain ``PYTHON_FUNCTION``), which the trace database imports
like any API trace. Counterpart of the reference's ``python -m rocprofsys`` (rocprofiler-systems
source/python/rocprofsys/__main__.py: ``--builtin``, ``--setup``, ``--full-filepath``, ``--label args file line``, function and
module ``include`` / ``exclude`` / ``restrict`` lists, ``--trace-c``; ``profiler.py``: the ``Profiler`` context manager, decorator
and ``runcall``). Filter semantics as there: ``restrict`` keeps only what matches, ``exclude`` drops what matches, ``include``
keeps what matches even when an exclude pattern matches too; patterns are regular expressions, searched.
"""
from __future__ import annotations

import argparse
import builtins
import functools
import os
import re
import sys
import threading
import time
from pathlib import Path
from typing import Callable, Dict, List, Optional, Sequence

DOMAIN = "PYTHON_FUNCTION"
_HERE = os.path.abspath(__file__)
_DEFAULT_EXCLUDE_FUNCTIONS = [r"^<(genexpr|listcomp|dictcomp|setcomp)>$"]
_DEFAULT_EXCLUDE_MODULES = [r"<frozen ", r"/threading\.py$", r"/contextlib\.py$"]


def _compile(patterns: Optional[Sequence[str]]) -> List[re.Pattern]:
    return [re.compile(p) for p in (patterns or [])]


class Profiler:
    """Records a range per call while active. ``records`` holds ``(label, tid, start_ns, end_ns, depth)``."""

    _active: Optional["Profiler"] = None

    def __init__(self, include_functions: Sequence[str] = (), exclude_functions: Sequence[str] = (), restrict_functions: Sequence[str] = (),
                 include_modules: Sequence[str] = (), exclude_modules: Sequence[str] = (), restrict_modules: Sequence[str] = (),
                 label: Sequence[str] = (), full_filepath: bool = False, trace_c: bool = False, min_duration_us: float = 0.0,
                 max_records: int = 2_000_000, backend: str = "auto"):
        self.inc_f, self.exc_f, self.res_f = _compile(include_functions), _compile([*_DEFAULT_EXCLUDE_FUNCTIONS, *exclude_functions]), _compile(restrict_functions)
        self.inc_m, self.exc_m, self.res_m = _compile(include_modules), _compile([*_DEFAULT_EXCLUDE_MODULES, *exclude_modules]), _compile(restrict_modules)
        self.label = tuple(label)
        self.full_filepath = full_filepath
        self.trace_c = trace_c
        self.min_ns = int(min_duration_us * 1000)
        self.max_records = max_records
        self.records: List[tuple] = []
        self.dropped = 0
        self._labels: Dict[object, Optional[str]] = {}     # code object (or C function) -> label, None = filtered out
        self._tls = threading.local()
        if backend not in ("auto", "monitoring", "setprofile"):
            raise ValueError("backend is auto, monitoring or setprofile")
        have = hasattr(sys, "monitoring")
        if backend == "monitoring" and not have:
            raise RuntimeError("sys.monitoring needs Python 3.12 or later")
        # Two ways to hear about calls. sys.monitoring (3.12+): events per code object that can be switched off for the code
        # objects the filters reject, so what is not traced costs nothing after its first call. sys.setprofile: one hook for
        # every call and return of every function, filtered inside the hook.
        self.backend = "monitoring" if (have and backend != "setprofile") else "setprofile"

    # ------------------------------------------------------------------ filters and labels
    def wanted(self, func: str, filename: str) -> bool:
        if filename == _HERE:
            return False
        included = any(r.search(func) for r in self.inc_f) or any(r.search(filename) for r in self.inc_m)
        if self.res_f and not any(r.search(func) for r in self.res_f):
            return False
        if self.res_m and not any(r.search(filename) for r in self.res_m):
            return False
        if included:
            return True
        return not (any(r.search(func) for r in self.exc_f) or any(r.search(filename) for r in self.exc_m))

    def _label_of(self, code) -> Optional[str]:
        func = getattr(code, "co_qualname", code.co_name)
        if not self.wanted(func, code.co_filename):
            return None
        tags = []
        if "file" in self.label:
            tags.append(code.co_filename if self.full_filepath else os.path.basename(code.co_filename))
        if "line" in self.label:
            tags.append(str(code.co_firstlineno))
        return func + (" [" + ":".join(tags) + "]" if tags else "")

    # ------------------------------------------------------------------ the hook
    def _hook(self, frame, event, arg):
        if event == "call":
            code = frame.f_code
            label = self._labels.get(code, self)
            if label is self:
                label = self._labels[code] = self._label_of(code)
            stack = self._stack()
            if label is not None and "args" in self.label:
                label = f"{label}({self._args(frame)})"
            stack.append((label, time.monotonic_ns()))
        elif event == "return":
            stack = self._stack()
            if stack:
                label, t0 = stack.pop()
                if label is not None:
                    self._finish(label, t0, len(stack))
        elif self.trace_c and event == "c_call":
            label = self._labels.get(arg, self)
            if label is self:
                name = getattr(arg, "__qualname__", getattr(arg, "__name__", "?"))
                mod = getattr(arg, "__module__", None) or ""
                full = f"{mod}.{name}" if mod else name
                label = self._labels[arg] = full if self.wanted(full, f"<builtin {mod}>") else None
            self._stack().append((label, time.monotonic_ns()))
        elif self.trace_c and event in ("c_return", "c_exception"):
            stack = self._stack()
            if stack:
                label, t0 = stack.pop()
                if label is not None:
                    self._finish(label, t0, len(stack))

    def _stack(self) -> list:
        try:
            return self._tls.stack
        except AttributeError:
            self._tls.stack = []
            self._tls.tid = threading.get_native_id()
            return self._tls.stack

    def _finish(self, label: str, t0: int, depth: int) -> None:
        t1 = time.monotonic_ns()
        if t1 - t0 < self.min_ns:
            return
        if len(self.records) >= self.max_records:
            self.dropped += 1
            return
        self.records.append((label, self._tls.tid, t0, t1, depth))

    @staticmethod
    def _args(frame) -> str:
        code = frame.f_code
        names = code.co_varnames[:code.co_argcount + code.co_kwonlyargcount]
        parts = []
        for n in names[:6]:
            try:
                v = repr(frame.f_locals.get(n))
            except Exception:  # noqa: BLE001  a repr that raises must not break the traced program
                v = "?"
            parts.append(f"{n}={v[:24]}")
        return ", ".join(parts)

    # ------------------------------------------------------------------ the monitoring callbacks
    def _mon_start(self, code, offset):
        label = self._labels.get(code, self)
        if label is self:
            label = self._labels[code] = self._label_of(code)
        if label is None:
            return sys.monitoring.DISABLE        # never again for this code object
        if "args" in self.label:
            label = f"{label}({self._args(sys._getframe(1))})"
        self._stack().append((label, time.monotonic_ns(), code))
        return None

    def _mon_end(self, code, offset, value):
        if self._labels.get(code, self) is None:
            return sys.monitoring.DISABLE
        self._mon_pop(code)
        return None

    def _mon_unwind(self, code, offset, exc):     # left by an exception: cannot be switched off per code object
        if self._labels.get(code) is not None:
            self._mon_pop(code)

    def _mon_pop(self, code) -> None:
        stack = self._stack()
        if stack and stack[-1][2] is code:
            label, t0, _ = stack.pop()
            self._finish(label, t0, len(stack))

    def _mon_call(self, code, offset, func, arg0):
        if self._labels.get(code, self) is None or type(func).__name__ not in ("builtin_function_or_method", "method_descriptor", "wrapper_descriptor"):
            return None
        label = self._labels.get(func, self)
        if label is self:
            name = getattr(func, "__qualname__", getattr(func, "__name__", "?"))
            mod = getattr(func, "__module__", None) or ""
            full = f"{mod}.{name}" if mod else name
            label = self._labels[func] = full if self.wanted(full, f"<builtin {mod}>") else None
        self._stack().append((label, time.monotonic_ns(), func))
        return None

    def _mon_c_end(self, code, offset, func, arg0):
        stack = self._stack()
        if stack and stack[-1][2] is func:
            label, t0, _ = stack.pop()
            if label is not None:
                self._finish(label, t0, len(stack))

    def _start_monitoring(self) -> None:
        m = sys.monitoring
        self._tool = m.PROFILER_ID
        if m.get_tool(self._tool) is not None:
            raise RuntimeError(f"another profiler ({m.get_tool(self._tool)}) already uses sys.monitoring")
        m.use_tool_id(self._tool, "b200-pytrace")
        E = m.events
        m.register_callback(self._tool, E.PY_START, self._mon_start)
        m.register_callback(self._tool, E.PY_RESUME, self._mon_start)
        m.register_callback(self._tool, E.PY_RETURN, self._mon_end)
        m.register_callback(self._tool, E.PY_YIELD, self._mon_end)
        m.register_callback(self._tool, E.PY_UNWIND, self._mon_unwind)
        events = E.PY_START | E.PY_RESUME | E.PY_RETURN | E.PY_YIELD | E.PY_UNWIND
        if self.trace_c:
            m.register_callback(self._tool, E.CALL, self._mon_call)
            m.register_callback(self._tool, E.C_RETURN, self._mon_c_end)
            m.register_callback(self._tool, E.C_RAISE, self._mon_c_end)
            events |= E.CALL | E.C_RETURN | E.C_RAISE
        m.set_events(self._tool, events)

    def _stop_monitoring(self) -> None:
        m = sys.monitoring
        m.set_events(self._tool, 0)
        for ev in (m.events.PY_START, m.events.PY_RESUME, m.events.PY_RETURN, m.events.PY_YIELD, m.events.PY_UNWIND, m.events.CALL, m.events.C_RETURN,
                   m.events.C_RAISE):
            m.register_callback(self._tool, ev, None)
        m.free_tool_id(self._tool)
        m.restart_events()          # what was switched off for this run is heard again by the next one

    # ------------------------------------------------------------------ control
    def start(self) -> "Profiler":
        if Profiler._active is not None:
            raise RuntimeError("a Python tracer is already active")
        Profiler._active = self
        if self.backend == "monitoring":
            self._start_monitoring()
            return self
        threading.setprofile(self._hook)
        if hasattr(threading, "setprofile_all_threads"):
            threading.setprofile_all_threads(self._hook)
        sys.setprofile(self._hook)
        return self

    def stop(self) -> "Profiler":
        if Profiler._active is self:
            if self.backend == "monitoring":
                self._stop_monitoring()
            else:
                sys.setprofile(None)
                threading.setprofile(None)
                if hasattr(threading, "setprofile_all_threads"):
                    threading.setprofile_all_threads(None)
            Profiler._active = None
            stack = getattr(self._tls, "stack", None)
            while stack:                     # ranges still open on this thread end now (the frames that called start())
                label, t0 = stack.pop()[:2]
                if label is not None:
                    self._finish(label, t0, len(stack))
        return self

    def __enter__(self) -> "Profiler":
        return self.start()

    def __exit__(self, *exc) -> None:
        self.stop()

    def __call__(self, func: Callable) -> Callable:
        @functools.wraps(func)
        def wrapper(*a, **k):
            if Profiler._active is not None:
                return func(*a, **k)
            with self:
                return func(*a, **k)
        return wrapper

    def runcall(self, func: Callable, *a, **k):
        with self:
            return func(*a, **k)

    def run_script(self, path: str, argv: Sequence[str]) -> None:
        """Runs ``path`` as ``__main__`` with ``argv`` under the tracer."""
        code = compile(Path(path).read_text(), path, "exec")
        globs = {"__name__": "__main__", "__file__": path, "__builtins__": builtins, "__package__": None}
        old_argv, old_path0 = sys.argv, sys.path[0] if sys.path else None
        sys.argv = [path, *argv]
        sys.path.insert(0, os.path.dirname(os.path.abspath(path)))
        try:
            with self:
                exec(code, globs)  # noqa: S102  this is what running a script means
        finally:
            sys.argv = old_argv
            if old_path0 is not None and sys.path and sys.path[0] != old_path0:
                sys.path.pop(0)

    # ------------------------------------------------------------------ output
    def write_csv(self, prefix: str) -> str:
        """``<prefix>.pytrace.<pid>.csv`` in the layout of the API traces; returns the path."""
        path = f"{prefix}.pytrace.{os.getpid()}.csv"
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        pid = os.getpid()
        with open(path, "w") as f:
            f.write('"Domain","Function","Process_Id","Thread_Id","Correlation_Id","Start_Timestamp","End_Timestamp","Depth"\n')
            for label, tid, t0, t1, depth in self.records:
                f.write(f'"{DOMAIN}","{label.replace(chr(34), chr(39))}",{pid},{tid},0,{t0},{t1},{depth}\n')
        return path

    def stats(self, top: int = 20) -> List[dict]:
        """Functions by inclusive time: ``{function, calls, total_ns, mean_ns, max_ns}``."""
        acc: Dict[str, list] = {}
        for label, _, t0, t1, _ in self.records:
            a = acc.setdefault(label, [0, 0, 0])
            a[0] += 1
            a[1] += t1 - t0
            a[2] = max(a[2], t1 - t0)
        rows = sorted(acc.items(), key=lambda kv: -kv[1][1])[:top]
        return [{"function": k, "calls": c, "total_ns": t, "mean_ns": t / c, "max_ns": m} for k, (c, t, m) in rows]


profile = Profiler()
"""A ready-made tracer for ``@profile`` and ``with profile:`` (what ``--builtin`` puts into the builtins)."""


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="pytrace", description=__doc__.split("\n\n")[0],
                                 epilog="usage: python -m rocm_systems_b200.tools.pytrace <options> -- <script> <script arguments>")
    ap.add_argument("-o", "--output", default=os.environ.get("B200COLL_TRACE_FILE", "pytrace"), metavar="PREFIX",
                    help="prefix of the output (default: the prefix the tracing launcher handed down, else ./pytrace)")
    ap.add_argument("-b", "--builtin", action="store_true", help="put `profile` into the builtins and trace only what the script marks with "
                    "@profile or `with profile:`")
    ap.add_argument("-s", "--setup", default=None, metavar="FILE", help="code to execute before the script, untraced")
    ap.add_argument("-F", "--full-filepath", action="store_true", help="whole file names in labels, not base names")
    ap.add_argument("--label", nargs="*", choices=("args", "file", "line"), default=[], help="add arguments, file name and / or line to the labels")
    ap.add_argument("-I", "--function-include", nargs="+", default=[], metavar="REGEX")
    ap.add_argument("-E", "--function-exclude", nargs="+", default=[], metavar="REGEX")
    ap.add_argument("-R", "--function-restrict", nargs="+", default=[], metavar="REGEX")
    ap.add_argument("-MI", "--module-include", nargs="+", default=[], metavar="REGEX", help="on the file name of the function's module")
    ap.add_argument("-ME", "--module-exclude", nargs="+", default=[], metavar="REGEX")
    ap.add_argument("-MR", "--module-restrict", nargs="+", default=[], metavar="REGEX")
    ap.add_argument("--trace-c", action="store_true", help="calls of C functions (builtins, extension modules) too")
    ap.add_argument("--min-duration-us", type=float, default=0.0, help="drop calls shorter than this")
    ap.add_argument("--max-records", type=int, default=2_000_000)
    ap.add_argument("--backend", choices=["auto", "monitoring", "setprofile"], default="auto",
                    help="monitoring (Python 3.12+): functions the filters reject cost nothing after their first call; setprofile: one hook for every call")
    ap.add_argument("--stats", action="store_true", help="print the functions by inclusive time when the script ends")
    ap.add_argument("--top", type=int, default=20)
    ap.add_argument("script", nargs=argparse.REMAINDER, help="-- script and its arguments")
    a = ap.parse_args(argv)
    words = a.script[1:] if a.script and a.script[0] == "--" else a.script
    if not words:
        ap.error("no script given (put it after --)")
    script = words[0]
    if not os.path.isfile(script):
        found = next((os.path.join(d, script) for d in os.environ.get("PATH", os.defpath).split(os.pathsep) if d and os.path.isfile(os.path.join(d, script))), None)
        if found is None:
            print(f"pytrace: cannot find script {script}", file=sys.stderr)
            return 1
        script = found
    global profile
    prof = Profiler(a.function_include, a.function_exclude, a.function_restrict, a.module_include, a.module_exclude, a.module_restrict, a.label,
                    a.full_filepath, a.trace_c, a.min_duration_us, a.max_records, a.backend)
    if a.setup:
        exec(compile(Path(a.setup).read_text(), a.setup, "exec"), {"__name__": "__setup__"})  # noqa: S102
    rc = 0
    import signal

    def ended(signum, frame):   # an ended run keeps what it traced: leave through the `finally` below
        raise SystemExit(128 + signum)

    if signal.getsignal(signal.SIGTERM) == signal.SIG_DFL:
        signal.signal(signal.SIGTERM, ended)
    try:
        if a.builtin:
            profile = prof
            builtins.profile = prof
            code = compile(Path(script).read_text(), script, "exec")
            old = sys.argv
            sys.argv = [script, *words[1:]]
            sys.path.insert(0, os.path.dirname(os.path.abspath(script)))
            try:
                exec(code, {"__name__": "__main__", "__file__": script, "__builtins__": builtins})  # noqa: S102
            finally:
                sys.argv = old
        else:
            prof.run_script(script, words[1:])
    except SystemExit as e:
        rc = e.code if isinstance(e.code, int) else (0 if e.code is None else 1)
    finally:
        prof.stop()
        path = prof.write_csv(a.output)
        print(f"pytrace: {len(prof.records)} calls in {path}" + (f" ({prof.dropped} dropped)" if prof.dropped else ""), file=sys.stderr)
        if a.stats:
            from .tracedb import format_table

            rows = prof.stats(a.top)
            if rows:
                print(format_table(list(rows[0].keys()), [list(r.values()) for r in rows]))
    return rc


if __name__ == "__main__":
    sys.exit(main())
