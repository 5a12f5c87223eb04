"""When a run stops making progress, say where: after a deadline every thread's Python stack is written out, followed by
what each registered communicator knows (asynchronous error state and the last error text, which for a bounded device wait
that ran out names the wait, the peer and the values seen).

The reference's system profiler arms the same kind of timer in CI: a thread that sends SIGHUP after a timeout so that all
thread backtraces are dumped (rocprofiler-systems source/lib/rocprof-sys/timeout.cpp:64-85).

    from rocm_systems_b200.utils import hang_dump
    hang_dump.arm(600, comms=[comm])        # once, at start; re-arm with hang_dump.kick() at every step
    ...
    hang_dump.disarm()
"""
from __future__ import annotations

import faulthandler
import sys
import threading
import time
from typing import Iterable, Optional, TextIO

_state = {"timer": None, "seconds": 0.0, "comms": [], "file": None, "exit": False}


def _report() -> None:
    out: TextIO = _state["file"] or sys.stderr
    out.write(f"\n=== hang_dump: no progress for {_state['seconds']:.0f} s ===\n")
    out.flush()
    faulthandler.dump_traceback(file=out, all_threads=True)
    for c in _state["comms"]:
        try:
            out.write(f"communicator rank {getattr(c, 'rank', '?')}/{getattr(c, 'nranks', '?')}: async error {c.async_error()}, last error: {c.last_error() or '-'}\n")
        except Exception as e:  # noqa: BLE001 - a report must not raise
            out.write(f"communicator {c!r}: {e}\n")
    out.flush()
    if _state["exit"]:
        import os

        os._exit(124)


def arm(seconds: float, comms: Optional[Iterable] = None, file: Optional[TextIO] = None, exit_after: bool = False) -> None:
    """Report after ``seconds`` without a ``kick()``. ``exit_after`` ends the process with status 124 after the report
    (for tests that must not outlive their budget)."""
    disarm()
    _state.update(seconds=float(seconds), comms=list(comms or []), file=file, exit=exit_after)
    kick()


def kick() -> None:
    """Progress was made: start the countdown again."""
    t = _state["timer"]
    if t is not None:
        t.cancel()
    if _state["seconds"] <= 0:
        return
    t = threading.Timer(_state["seconds"], _report)
    t.daemon = True
    t.start()
    _state["timer"] = t


def disarm() -> None:
    t = _state["timer"]
    if t is not None:
        t.cancel()
    _state["timer"] = None
    _state["seconds"] = 0.0


class watch:
    """``with hang_dump.watch(300, comms=[comm]):`` arms on entry and disarms on exit."""

    def __init__(self, seconds: float, comms: Optional[Iterable] = None, file: Optional[TextIO] = None, exit_after: bool = False):
        self.args = (seconds, comms, file, exit_after)

    def __enter__(self) -> "watch":
        arm(*self.args)
        return self

    def __exit__(self, *exc) -> None:
        disarm()


def _selftest() -> int:  # python -m rocm_systems_b200.utils.hang_dump
    class Fake:
        rank, nranks = 1, 4

        def async_error(self):
            return 6

        def last_error(self):
            return "wait BARRIER for rank 3 gave up: expected 12, saw 11"

    arm(0.2, comms=[Fake()])
    time.sleep(0.6)
    disarm()
    return 0


if __name__ == "__main__":
    sys.exit(_selftest())
