"""Range and point markers that land in the same trace as collectives and kernels.

Python face of ``b200tx`` (csrc/include/b200coll/markers.h); the analogue of the reference's
``roctx`` Python binding (rocprofiler-sdk/source/lib/python/roctx). Recording is off until
``enable()`` is called or ``B200COLL_TRACE=1`` is in the environment.

    from rocm_systems_b200.utils import markers
    with markers.range("step 12"):
        ...
"""
from __future__ import annotations

import contextlib
import ctypes
from typing import Iterator, List

from .. import _lib


class _Record(ctypes.Structure):
    _fields_ = [("id", ctypes.c_uint64), ("begin_ns", ctypes.c_uint64), ("end_ns", ctypes.c_uint64), ("tid", ctypes.c_uint32),
                ("depth", ctypes.c_uint32), ("message", ctypes.c_char * 96)]


_ready = False


def _l():
    global _ready
    lib = _lib.load()
    if not _ready:
        lib.b200txMark.argtypes = [ctypes.c_char_p]
        lib.b200txRangePush.argtypes = [ctypes.c_char_p]
        lib.b200txRangeStart.argtypes = [ctypes.c_char_p]
        lib.b200txRangeStart.restype = ctypes.c_uint64
        lib.b200txRangeStop.argtypes = [ctypes.c_uint64]
        lib.b200txRangeAt.argtypes = [ctypes.c_char_p, ctypes.c_uint64, ctypes.c_uint64]
        lib.b200txRangeAt.restype = ctypes.c_uint64
        lib.b200txEnable.argtypes = [ctypes.c_int]
        lib.b200txGet.argtypes = [ctypes.c_void_p, ctypes.c_uint64]
        lib.b200txGet.restype = ctypes.c_uint64
        lib.b200collBuildInfo.restype = ctypes.c_char_p
        _ready = True
    return lib


def enable(on: bool = True) -> None:
    _l().b200txEnable(1 if on else 0)


def mark(message: str) -> None:
    _l().b200txMark(message.encode())


def range_push(message: str) -> int:
    return int(_l().b200txRangePush(message.encode()))


def range_at(message: str, begin_ns: int, end_ns: int) -> int:
    """Records a range that is already over (times on ``time.monotonic_ns()``'s clock); returns its id, 0 when recording is off."""
    return int(_l().b200txRangeAt(message.encode(), int(begin_ns), int(end_ns)))


def range_pop() -> int:
    return int(_l().b200txRangePop())


def range_start(message: str) -> int:
    return int(_l().b200txRangeStart(message.encode()))


def range_stop(range_id: int) -> None:
    _l().b200txRangeStop(range_id)


@contextlib.contextmanager
def range(message: str) -> Iterator[None]:  # noqa: A001 - mirrors the C name
    range_push(message)
    try:
        yield
    finally:
        range_pop()


def records() -> List[dict]:
    lib = _l()
    n = int(lib.b200txGet(None, 0))
    if n == 0:
        return []
    buf = (_Record * n)()
    n = min(n, int(lib.b200txGet(buf, n)))
    return [{"id": r.id, "begin_ns": r.begin_ns, "end_ns": r.end_ns, "tid": r.tid, "depth": r.depth,
             "message": r.message.decode(errors="replace")} for r in buf[:n]]


def clear() -> None:
    _l().b200txClear()


def write_csv(path: str, pid: int | None = None) -> int:
    """Writes the finished ranges in the marker-trace CSV layout; returns the row count."""
    import os

    rows = records()
    pid = os.getpid() if pid is None else pid
    with open(path, "w") as f:
        f.write('"Domain","Function","Process_Id","Thread_Id","Correlation_Id","Start_Timestamp","End_Timestamp","Depth"\n')
        for r in rows:
            msg = r["message"].replace('"', "'")
            f.write(f'"MARKER_API","{msg}",{pid},{r["tid"]},{r["id"]},{r["begin_ns"]},{r["end_ns"]},{r["depth"]}\n')
    return len(rows)


def install_path() -> dict:
    """``{"library": file the native library was loaded from, "prefix": the directory above its lib/}``."""
    lib = _l()
    lib.b200collGetInstallPath.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t]
    a, b = ctypes.create_string_buffer(4096), ctypes.create_string_buffer(4096)
    if lib.b200collGetInstallPath(a, 4096, b, 4096) != 0:
        raise RuntimeError("the library cannot tell where it was loaded from")
    return {"library": a.value.decode(), "prefix": b.value.decode()}


def build_info() -> str:
    return _l().b200collBuildInfo().decode()
