"""Host-side rendezvous: rounds, descriptor passing and failure notices, as CPU processes.

The reference tests multi-process plumbing with fork()ed pairs and env-keyed fault injection
(rocr-runtime/rocrtst/suites/functional/ipc.cc:141-255); these tests do the same against the
bootstrap service, with no GPU involved.
"""
import ctypes
import multiprocessing as mp
import os
import time

import pytest

from rocm_systems_b200 import _lib


def _worker(rank, n, idbytes, q, env, scenario):
    os.environ.update(env)
    lib = _lib.load()
    lib.b200collRefreshFlags()
    uid = _lib.UniqueId()
    ctypes.memmove(ctypes.addressof(uid), idbytes, 128)
    h = ctypes.c_void_p()
    rc = lib.b200collBootCreate(ctypes.byref(uid), rank, n, ctypes.byref(h))
    if rc != 0:
        q.put((rank, "init", rc))
        return
    try:
        if scenario == "allgather":
            send = (ctypes.c_int * 4)(rank, rank * 10, rank * 100, 7)
            recv = (ctypes.c_int * (4 * n))()
            for _ in range(3):
                rc = lib.b200collBootAllGather(h, send, recv, 16)
                assert rc == 0
            rc = lib.b200collBootBarrier(h)
            q.put((rank, "ok", list(recv)))
        elif scenario == "fd":
            # every rank passes a pipe's read end to its right neighbour, then writes to it
            r, w = os.pipe()
            right, left = (rank + 1) % n, (rank - 1) % n
            assert lib.b200collBootSendFd(h, right, r, 42) == 0
            got = ctypes.c_int(-1)
            assert lib.b200collBootRecvFd(h, left, 42, ctypes.byref(got)) == 0
            os.write(w, f"from{rank}".encode())
            assert lib.b200collBootBarrier(h) == 0
            data = os.read(got.value, 64).decode()
            q.put((rank, "ok", data))
        elif scenario == "die":
            if rank == 1:
                time.sleep(0.2)
                os._exit(0)  # leaves without a goodbye
            rc = lib.b200collBootBarrier(h)
            q.put((rank, "rc", rc))
        elif scenario == "notice":
            if rank == 1:
                time.sleep(0.2)
                os._exit(0)
            who = -1
            for _ in range(100):
                who = lib.b200collBootPeerFailed(h)
                if who >= 0:
                    break
                time.sleep(0.05)
            q.put((rank, "who", who))
        elif scenario == "silent":
            rc = lib.b200collBootBarrier(h)
            q.put((rank, "rc", rc))
    finally:
        lib.b200collBootClose(h, 1)


def _run(n, scenario, env=None):
    ctx = mp.get_context("spawn")
    lib = _lib.load()
    uid = _lib.UniqueId()
    assert lib.ncclGetUniqueId(ctypes.byref(uid)) == 0
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, n, ctypes.string_at(ctypes.addressof(uid), 128), q, env or {}, scenario)) for r in range(n)]
    for p in procs:
        p.start()
    out = {}
    deadline = time.time() + 60
    expected = n if scenario not in ("die", "notice") else n - 1
    while len(out) < expected and time.time() < deadline:
        try:
            r, kind, val = q.get(timeout=1)
            out[r] = (kind, val)
        except Exception:
            pass
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.kill()
    return out


def test_allgather_rounds():
    out = _run(3, "allgather")
    assert len(out) == 3
    for r in range(3):
        kind, vals = out[r]
        assert kind == "ok"
        for s in range(3):
            assert vals[4 * s:4 * s + 4] == [s, s * 10, s * 100, 7]


def test_descriptor_passing():
    out = _run(3, "fd")
    assert len(out) == 3
    for r in range(3):
        assert out[r] == ("ok", f"from{(r - 1) % 3}")


def test_rank_that_exits_is_reported_in_round():
    out = _run(3, "die", env={"B200COLL_BOOTSTRAP_TIMEOUT_MS": "8000"})
    assert set(out) == {0, 2}
    for r in (0, 2):
        kind, rc = out[r]
        assert kind == "rc" and rc == 6  # ncclRemoteError


def test_rank_that_exits_is_noticed_without_a_round():
    out = _run(2, "notice")
    assert out[0] == ("who", 1)


def test_silent_rank_times_out_cleanly():
    env = {"B200COLL_BOOTSTRAP_TIMEOUT_MS": "1500", "B200COLL_FAIL_KEY": "boot_skip_round_rank1"}
    t0 = time.time()
    out = _run(2, "silent", env=env)
    assert time.time() - t0 < 30
    assert out[0][0] == "rc" and out[0][1] in (2, 6)  # system (timeout) or remote error


def _comm_id_worker(rank, n, comm_id, q):
    os.environ["B200COLL_COMM_ID"] = comm_id
    lib = _lib.load()
    lib.b200collRefreshFlags()
    uid = _lib.UniqueId()
    if rank:
        time.sleep(0.05 * rank)                       # not everybody asks at the same instant
    rc = lib.ncclGetUniqueId(ctypes.byref(uid))       # every rank asks for "the" id itself
    if rc != 0:
        q.put((rank, "id", rc))
        return
    h = ctypes.c_void_p()
    rc = lib.b200collBootCreate(ctypes.byref(uid), rank, n, ctypes.byref(h))
    if rc != 0:
        q.put((rank, "init", rc))
        return
    send = (ctypes.c_int * 1)(100 + rank)
    recv = (ctypes.c_int * n)()
    rc = lib.b200collBootAllGather(h, send, recv, 4)
    assert lib.b200collBootBarrier(h) == 0
    q.put((rank, "ok", (ctypes.string_at(ctypes.addressof(uid), 128).hex(), list(recv), rc)))
    lib.b200collBootClose(h, 1)


def test_comm_id_gives_every_rank_the_same_id_without_an_exchange():
    """With COMM_ID=ip:port nobody has to ship the unique id around: every rank derives the same id
    from the string, and whichever rank gets the port serves the rendezvous."""
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    n = 3
    procs = [ctx.Process(target=_comm_id_worker, args=(r, n, f"127.0.0.1:{port}", q)) for r in range(n)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert all(r[1] == "ok" for r in res), res
    ids = {r[2][0] for r in res}
    assert len(ids) == 1
    assert all(r[2][1] == [100, 101, 102] and r[2][2] == 0 for r in res)
