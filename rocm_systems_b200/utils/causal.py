"""Progress points for causal profiling from Python. When the program runs under ``libb200causal.so``
(``python -m rocm_systems_b200.tools.causal run -- python train.py``), ``progress("step")`` counts one visit of a
throughput point and ``begin`` / ``end`` bracket one item of a latency point; without the library they do nothing. The
experiments themselves select native functions (``-B`` names the shared objects in scope, e.g. ``libb200coll`` or an
extension module), since it is native code whose speed-up the pauses emulate.

Counterpart of the reference's user macros ``ROCPROFSYS_CAUSAL_PROGRESS`` / ``_BEGIN`` / ``_END``
(rocprofiler-systems source/lib/rocprof-sys-user/rocprofiler-systems/causal.h) and of its Python binding's
``rocprofsys.user`` calls."""
from __future__ import annotations

import ctypes
from contextlib import contextmanager
from typing import Optional

_fns: Optional[dict] = None


def _load() -> dict:
    global _fns
    if _fns is None:
        _fns = {}
        try:
            me = ctypes.CDLL(None)
            for name in ("b200causalProgress", "b200causalBegin", "b200causalEnd", "b200causalActive"):
                fn = getattr(me, name)
                if name != "b200causalActive":
                    fn.argtypes = [ctypes.c_char_p]
                    fn.restype = None
                else:
                    fn.restype = ctypes.c_int
                _fns[name] = fn
        except (OSError, AttributeError):
            _fns = {}
    return _fns


def active() -> bool:
    """True while the causal profiler is loaded into this process and sampling."""
    fn = _load().get("b200causalActive")
    return bool(fn()) if fn else False


def progress(name: str = "step") -> None:
    fn = _load().get("b200causalProgress")
    if fn:
        fn(name.encode())


def begin(name: str) -> None:
    fn = _load().get("b200causalBegin")
    if fn:
        fn(name.encode())


def end(name: str) -> None:
    fn = _load().get("b200causalEnd")
    if fn:
        fn(name.encode())


@contextmanager
def item(name: str):
    """``with item("batch"):`` one item in flight of the latency point ``name``."""
    begin(name)
    try:
        yield
    finally:
        end(name)
