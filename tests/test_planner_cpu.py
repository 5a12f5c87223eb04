"""The collective planner without a device: which algorithm, how many CTAs and how many pipeline
chunks a message gets, under the built-in thresholds, the environment and a tuning file."""
import ctypes
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
AR, RS, RED, AG, BC = range(5)
LL, P2P, NVLS = 1, 2, 3
F32, SUM, MAX = 7, 0, 2

CODE = """
import ctypes, json, sys
from rocm_systems_b200 import _lib
lib = _lib.load()
class Info(ctypes.Structure):
    _fields_ = [("algo", ctypes.c_int), ("ctas", ctypes.c_int), ("direct", ctypes.c_int), ("chunks", ctypes.c_ulonglong)]
lib.b200collPlanDry.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.POINTER(Info)]
out = []
for nranks, nvls, kind, count, dt, op in json.loads(sys.argv[1]):
    i = Info()
    rc = lib.b200collPlanDry(nranks, nvls, kind, count, dt, op, ctypes.byref(i))
    out.append([rc, i.algo, i.ctas, i.direct, i.chunks])
print(json.dumps(out))
"""


def plan(cases, env=None):
    e = dict(os.environ, PYTHONPATH=str(ROOT))
    for k in list(e):
        if k.startswith(("B200COLL_", "NCCL_")):
            del e[k]
    e.update(env or {})
    p = subprocess.run([sys.executable, "-c", CODE, json.dumps(cases)], env=e, capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr
    return json.loads(p.stdout.strip().splitlines()[-1])


def test_builtin_choices():
    MiB = 1 << 20
    r = plan([
        [8, 1, AR, 1024, F32, SUM],            # 4 KiB: flag-in-data
        [8, 1, AR, 128 * 1024, F32, SUM],      # 512 KiB: still flag-in-data between eight ranks
        [8, 1, AR, 128 * 1024 + 4, F32, SUM],  # just above: in-switch
        [8, 1, AR, 64 * MiB // 4, F32, MAX],   # max is not an in-switch operation: peer loads
        [2, 1, AR, 64 * MiB // 4, F32, SUM],   # two ranks: peer loads move fewer bytes than the switch
        [8, 0, AR, 64 * MiB // 4, F32, SUM],   # no multicast: peer loads
        [8, 1, AG, MiB, F32, SUM],             # copies never reduce in the switch
        [8, 1, AR, 8, 6, SUM],                 # fp16 is 6: tiny, flag-in-data
        [2, 1, AR, 2 * MiB // 4, F32, SUM],    # between two ranks flag-in-data carries up to 2 MiB, on up to 64 CTAs (within the communicator's budget)
        [2, 1, AR, 2 * MiB // 4 + 4, F32, SUM],
        [8, 1, RS, 64 * 1024, F32, SUM],       # reduce-scatter / all-gather: flag-in-data for slices up to 4 x 512 KiB / 8 ranks
        [8, 1, RS, 64 * 1024 + 4, F32, SUM],
        [8, 1, AG, 64 * 1024, F32, SUM],
        [8, 1, AG, 64 * 1024 + 4, F32, SUM],
        [2, 1, AG, 2 * MiB // 4, F32, SUM],    # two ranks: slices up to 2 MiB
    ])
    assert [x[0] for x in r] == [0] * 15
    assert [x[1] for x in r] == [LL, LL, NVLS, P2P, P2P, P2P, P2P, LL, LL, P2P, LL, NVLS, LL, P2P, LL]
    assert r[0][2] == 1 and r[1][2] == 32 and r[8][2] == 32   # 512 KiB between 8 ranks: 7 MiB of lines per rank, one CTA per 64 KiB of them;          # 64 by size, bounded by the CTA budget of the planning communicator (32)
    assert plan([[2, 1, AR, 2 * MiB // 4, F32, SUM]], {"B200COLL_MAX_CTAS": "64"})[0][2] == 64
    assert all(x[3] == 0 for x in r)           # nothing is in a registered window here


def test_pipeline_chunks_are_equalised():
    MiB = 1 << 20
    r = plan([
        [8, 1, AR, 8 * MiB // 4, F32, SUM],        # 8 MiB: one chunk
        [8, 1, AR, 16 * MiB // 4, F32, SUM],       # 16 MiB: still one chunk (a chunk costs its barriers; none below 32 MiB)
        [8, 1, AR, 80 * 1000 * 1000 // 4, F32, SUM],   # 80 MB: an eighth is below the 32 MiB minimum -> three equal chunks
        [8, 1, AR, 1024 * MiB // 4, F32, SUM],     # 1 GiB: a staging half (64 MiB) caps the chunk: 16
        [8, 1, RS, 128 * MiB // 4, F32, SUM],      # per-rank slice 128 MiB -> staged 1 GiB -> 8 MiB per slice and chunk: 16
        [8, 1, AG, 200 * MiB // 4, F32, SUM],      # copies are chunked by the staging half only: ceil(200 / 64) = 4
    ])
    assert [x[4] for x in r] == [1, 1, 3, 16, 16, 4]
    off = plan([[8, 1, AR, 1024 * MiB // 4, F32, SUM]], {"B200COLL_PIPELINE_CHUNK": "0"})
    assert off[0][4] == 16                         # 64 MiB halves either way at this size
    small = plan([[8, 1, AR, 32 * MiB // 4, F32, SUM]], {"B200COLL_PIPELINE_CHUNK": "1M"})
    assert small[0][4] == 32


def test_environment_and_cta_bounds():
    MiB = 1 << 20
    base = plan([[8, 1, AR, 64 * MiB // 4, F32, SUM]])[0]
    assert base[1] == NVLS and base[2] == 32       # the default upper bound
    forced = plan([[8, 1, AR, 64 * MiB // 4, F32, SUM]], {"NCCL_ALGO": "P2P", "NCCL_MAX_CTAS": "8"})[0]
    assert forced[1] == P2P and forced[2] == 8
    no_nvls = plan([[8, 1, AR, 64 * MiB // 4, F32, SUM]], {"NCCL_NVLS_ENABLE": "0"})[0]
    assert no_nvls[1] == P2P
    # a forced algorithm that cannot serve the call falls back: flag-in-data does not do 64 MiB
    assert plan([[8, 1, AR, 64 * MiB // 4, F32, SUM]], {"B200COLL_ALGO": "ll"})[0][1] == NVLS


def test_tuning_file_wins_over_thresholds(tmp_path):
    MiB = 1 << 20
    t = tmp_path / "tune.json"
    t.write_text(json.dumps({"entries": [{"coll": "all_reduce", "nranks": 8, "max_bytes": MiB, "algo": "p2p", "ctas": 5},
                                         {"coll": "all_reduce", "nranks": 4, "max_bytes": 1 << 40, "algo": "ll"},
                                         {"coll": "all_reduce", "max_bytes": 1 << 40, "algo": "nvls"}]}))
    r = plan([[8, 1, AR, 1024, F32, SUM], [8, 1, AR, 4 * MiB // 4, F32, SUM], [8, 1, RS, 1024, F32, SUM]], {"B200COLL_TUNING_FILE": str(t)})
    assert r[0][1] == P2P and r[0][2] == 5        # first row covers 4 KiB
    assert r[1][1] == NVLS                         # beyond the first row; the 4-rank row is skipped at 8 ranks
    assert r[2][1] == LL                           # no reduce_scatter rows: built-in choice (slices of 4 KiB: flag-in-data)
    assert plan([[0, 1, AR, 4, F32, SUM]])[0][0] == 4   # nranks 0: invalid argument


def test_planner_invariants_over_random_messages():
    """Properties that hold for every message: a valid algorithm, a CTA count inside the limits, at least one chunk,
    flag-in-data only for small all-reduces, the in-switch path only where the switch can add (float sums, more than two
    ranks, multicast present), and chunk counts that grow with the message."""
    import random

    rng = random.Random(11)
    cases = []
    for _ in range(400):
        nranks = rng.choice([2, 3, 4, 8])
        kind = rng.choice([AR, RS, RED, AG, BC])
        count = rng.choice([1, 3, 17, 1000, 4099, 16384, 16385, 70001, 1 << 20, (1 << 22) + 5, 1 << 26, (1 << 28) + 1, 1 << 29])
        cases.append([nranks, rng.choice([0, 1]), kind, count, rng.choice([F32, 2, 9, 0]), rng.choice([SUM, MAX])])   # 2: int32, 9: bf16, 0: int8
    res = plan(cases)
    for (nranks, nvls, kind, count, dt, op), (rc, algo, ctas, direct, chunks) in zip(cases, res):
        es = {F32: 4, 2: 4, 9: 2, 0: 1}[dt]
        nbytes = count * es
        assert rc == 0 and algo in (LL, P2P, NVLS) and 1 <= ctas <= 128 and direct == 0, (nranks, kind, count, algo, ctas, chunks)
        assert (chunks == 0) if algo == LL else (chunks >= 1), (nranks, kind, count, algo, chunks)      # flag-in-data uses no staging
        if algo == LL:
            limit = {2: 2 << 20, 3: 2 << 20, 4: 1 << 20, 8: 512 << 10}[nranks]
            assert kind in (AR, RS, AG) and nbytes <= (limit if kind == AR or nranks == 2 else min(limit, limit * 4 // nranks))
        if algo == NVLS:
            assert nvls == 1
            if kind in (AR, RS, RED):
                assert nranks > 2 and op == SUM and dt in (F32, 9)
        if nbytes <= 1 << 20 and algo != LL:
            assert chunks == 1
    # more bytes never means fewer chunks (same collective, ranks and type)
    sizes = [1 << k for k in range(10, 30)]
    for kind in (AR, RS, AG):
        r = plan([[8, 1, kind, s, F32, SUM] for s in sizes])
        chunk_counts = [x[4] for x in r]
        assert chunk_counts == sorted(chunk_counts) and chunk_counts[-1] > 1


def test_all_to_all_takes_one_of_three_paths():
    """ncclAllToAll on ordinary buffers, by bytes per pair: the flag-in-data kernel up to the slice limit, the staged kernel by peer
    stores from 1 MiB (steps = slots of a staging half), the send/recv FIFOs in between; the switch moves with the environment."""
    A2A, FIFO = 5, 4
    MiB = 1 << 20
    r = plan([
        [8, 1, A2A, 64 * 1024, F32, SUM],          # 256 KiB per pair between eight ranks: flag-in-data
        [8, 1, A2A, 64 * 1024 + 4, F32, SUM],      # just above: FIFOs
        [8, 1, A2A, MiB // 4, F32, SUM],           # 1 MiB per pair: staged
        [8, 1, A2A, 64 * MiB // 4, F32, SUM],      # 64 MiB per pair: 8 MiB slots -> 8 steps
        [2, 1, A2A, 2 * MiB // 4, F32, SUM],       # two ranks: flag-in-data up to 2 MiB per pair
        [2, 1, A2A, 64 * MiB // 4, F32, SUM],      # 32 MiB slots -> 2 steps
    ])
    assert [x[0] for x in r] == [0] * 6
    assert [x[1] for x in r] == [LL, FIFO, P2P, P2P, LL, P2P]
    assert [x[4] for x in r] == [0, 1, 1, 8, 0, 2]
    off = plan([[8, 1, A2A, 64 * MiB // 4, F32, SUM]], {"B200COLL_A2A_STAGED_MIN": "1G"})[0]
    assert off[1] == FIFO and off[4] == 128      # 512 KiB FIFO slots
    always = plan([[8, 1, A2A, 64 * 1024 + 4, F32, SUM]], {"B200COLL_A2A_STAGED_MIN": "0"})[0]
    assert always[1] == P2P
