"""Host-side failure detection and group re-formation for training loops.

A rank can be lost in two ways: it leaves between steps (says so in the store), or it stops
beating (crash, hang). Survivors learn of either on the host, at a step boundary and before their
next launch — nothing here waits on a GPU. They then abort / destroy the old process group, agree
on the survivor list through the store, build a new group without the lost ranks and reload the
last complete checkpoint (``utils/checkpoint.py`` re-shards it to the new world size).

The reference's runtime turns device faults and hangs into an error on the host and an abort
(runtime.cpp:1740-1944 handlers, default_signal.cpp:77-112 abort timeout); rccl-tests polls
``ncclCommGetAsyncError`` and aborts the communicator (common.cpp:586-611). This module is the
layer above: who is alive, and how the job carries on.

    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0))
    hb = Heartbeat(store, rank, world, interval=0.2, timeout=2.0).start()
    ...
    lost = hb.lost()                       # at a step boundary
    if lost:
        rank, world = reform_group(store, hb, generation=1, backend="gloo")
"""
from __future__ import annotations

import threading
import time
from datetime import timedelta
from typing import List, Optional, Tuple

import torch.distributed as dist


class Heartbeat:
    """Every rank writes a counter to ``hb/<rank>`` every ``interval`` seconds; a rank whose counter
    has not moved for ``timeout`` seconds, or that wrote ``left/<rank>``, counts as lost."""

    def __init__(self, store, rank: int, world: int, interval: float = 0.5, timeout: float = 5.0):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout = interval, timeout
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._seen = {r: (-1, time.monotonic()) for r in range(world)}
        self._beats = 0
        self.members = list(range(world))

    def _beat(self) -> None:
        self._beats += 1
        self.store.set(f"hb/{self.rank}", str(self._beats))

    def start(self) -> "Heartbeat":
        self._beat()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self._beat()
            except Exception:  # noqa: BLE001 - the store went away: the job is ending
                return

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def leave(self) -> None:
        """Announce a clean exit (between steps, with nothing in flight) and stop beating."""
        self.store.set(f"left/{self.rank}", "1")
        self.stop()

    def _count(self, key: str) -> Optional[str]:
        try:
            if not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:  # noqa: BLE001
            return None

    def lost(self) -> List[int]:
        """Ranks of the current membership that left or stopped beating."""
        now = time.monotonic()
        out = []
        for r in self.members:
            if r == self.rank:
                continue
            if self._count(f"left/{r}") is not None:
                out.append(r)
                continue
            v = self._count(f"hb/{r}")
            last, when = self._seen[r]
            cur = int(v) if v is not None else -1
            if cur != last:
                self._seen[r] = (cur, now)
            elif now - when > self.timeout:
                out.append(r)
        return out


def agree_survivors(store, hb: Heartbeat, generation: int, settle: float = 1.0) -> List[int]:
    """Every survivor proposes the members it still sees; the new membership is the intersection of
    all proposals from ranks that are in every proposal (so one slow detector cannot split the job).
    Returns the sorted list of old ranks that form the next group."""
    mine = [r for r in hb.members if r not in set(hb.lost())]
    store.set(f"gen{generation}/proposal/{hb.rank}", ",".join(map(str, mine)))
    # Survivors notice a loss at slightly different times; wait several heartbeat timeouts for the
    # proposals of everyone this rank still believes in before deciding without them.
    deadline = time.monotonic() + max(settle, 5 * hb.timeout)
    proposals = {}
    while time.monotonic() < deadline:
        proposals = {}
        for r in mine:
            key = f"gen{generation}/proposal/{r}"
            try:
                if store.check([key]):
                    proposals[r] = [int(x) for x in store.get(key).decode().split(",") if x]
            except Exception:  # noqa: BLE001
                pass
        if len(proposals) == len(mine):
            break
        time.sleep(0.05)
    alive = set(proposals)  # who answered
    for members in proposals.values():
        alive &= set(members)
    return sorted(alive)


def reform_group(store, hb: Heartbeat, generation: int, backend: str = "gloo", timeout_s: float = 60.0) -> Tuple[int, int]:
    """Tear down the current default process group and build generation ``generation`` from the
    survivors. Returns this rank's new ``(rank, world)``. A rank that finds itself outside the new
    membership gets ``(-1, 0)`` and should exit."""
    survivors = agree_survivors(store, hb, generation)
    if dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001 - a broken group may refuse a clean shutdown
            pass
    if hb.rank not in survivors:
        return -1, 0
    new_rank, new_world = survivors.index(hb.rank), len(survivors)
    prefix = dist.PrefixStore(f"gen{generation}", store)
    dist.init_process_group(backend, store=prefix, rank=new_rank, world_size=new_world, timeout=timedelta(seconds=timeout_s))
    hb.members = survivors
    return new_rank, new_world
