"""Sequential emulation of the staged kernels' byte arithmetic (csrc/coll/kernels.cuh) against numpy:
the all-reduce / reduce-scatter path (copy-in of every slice, reduction of slice `rank` out of every
rank's staging, delivery, copy-out) and the all-gather path, with the host's equalised chunking
(csrc/coll/enqueue.cc). Every output byte must be produced exactly once and be right, for ragged
sizes, any lane count and any rank count. Ordering between lanes and ranks is the business of
tests/test_protocol_model_cpu.py."""
import random

import numpy as np

U = 16


def ceil_div(a, b):
    return (a + b - 1) // b


def host_chunking(nbytes, full_cap, pipe_chunk=None):
    """cap and chunk count as planInternal computes them (pipe_chunk: the reduce kinds' pipeline chunk, or None)."""
    cap_max = full_cap
    if pipe_chunk is not None and 16 <= pipe_chunk < cap_max:
        cap_max = pipe_chunk
    k = ceil_div(nbytes, cap_max)
    cap = (ceil_div(nbytes, k) + 15) & ~15
    cap = min(cap, cap_max)
    return cap, ceil_div(nbytes, cap)


def lane_range(units, per_lane, b):
    lo = min(b * per_lane, units)
    return lo, min(lo + per_lane, units)


def emulate_reduce(n, lanes, count, stage_bytes, kind, rng):
    es = 4
    total = count * es                                     # the message (all-reduce) or one rank's slice (reduce-scatter)
    is_rs = kind == "rs"
    full_cap = ((stage_bytes // n) & ~15) if is_rs else stage_bytes
    staged = total * n if is_rs else total
    pipe = None
    if staged >= 4 * U * n:                                # stand-in for "large enough to pipeline"
        chunk = max(2 * U * n, ceil_div(staged, 8))
        pipe = ((chunk // n) & ~15) if is_rs else (chunk + 15) & ~15
    cap, chunks = host_chunking(total, full_cap, pipe)
    cap_units = ceil_div(cap, U)
    su = cap_units if is_rs else ceil_div(cap_units, n)
    per_lane = ceil_div(su, lanes)
    send = [rng.integers(-9, 10, size=(n * count if is_rs else count)).astype(np.int32) for _ in range(n)]
    stage = [np.zeros((2, stage_bytes + 64), dtype=np.uint8) for _ in range(n)]
    out = [np.zeros(count, dtype=np.int32) for _ in range(n)]
    hits = [np.zeros(count, dtype=np.int32) for _ in range(n)]

    def slice_bytes(cb, s):
        if is_rs:
            return cb
        lo = s * su * U
        return max(0, min(cb - lo, su * U))

    def slice_stage(s):
        return s * cap if is_rs else s * su * U

    done_chunks, half, off = 0, 0, 0
    while off < total:
        cb = min(cap, total - off)
        # copy-in
        for r in range(n):
            sb_all = send[r].view(np.uint8)
            for b in range(lanes):
                for s in range(n):
                    sb = slice_bytes(cb, s)
                    lo, hi = lane_range(ceil_div(sb, U), per_lane, b)
                    if lo < hi:
                        nb = min(hi * U, sb) - lo * U
                        src0 = (s * count * es + off if is_rs else off + s * su * U) + lo * U
                        d0 = slice_stage(s) + lo * U
                        assert d0 + nb <= stage_bytes, "staging overflow"
                        stage[r][half, d0:d0 + nb] = sb_all[src0:src0 + nb]
        # reduce slice r; all-reduce writes the result back into every rank's staging
        results = []
        for r in range(n):
            sb = slice_bytes(cb, r)
            for b in range(lanes):
                lo, hi = lane_range(ceil_div(sb, U), per_lane, b)
                for u in range(lo, hi):
                    st = slice_stage(r) + u * U
                    acc = sum(stage[p][half, st:st + U].view(np.int32).astype(np.int64) for p in range(n)).astype(np.int32)
                    if is_rs:
                        e0 = (off + u * U) // es
                        for kk in range(U // es):
                            if off + u * U + (kk + 1) * es <= total:
                                out[r][e0 + kk] = acc[kk]
                                hits[r][e0 + kk] += 1
                    else:
                        results.append((st, acc.copy()))
        if not is_rs:
            for st, acc in results:                        # applied after all reads: a slice is read only by its reducer
                for p in range(n):
                    stage[p][half, st:st + U] = acc.view(np.uint8)
            # copy-out
            for r in range(n):
                ob = out[r].view(np.uint8)
                for b in range(lanes):
                    for s in range(n):
                        sb = slice_bytes(cb, s)
                        lo, hi = lane_range(ceil_div(sb, U), per_lane, b)
                        if lo < hi:
                            nb = min(hi * U, sb) - lo * U
                            d0 = off + s * su * U + lo * U
                            ob[d0:d0 + nb] = stage[r][half, slice_stage(s) + lo * U: slice_stage(s) + lo * U + nb]
                            hits[r].view(np.uint8)[d0:d0 + nb] += 1
        off += cap
        half ^= 1
        done_chunks += 1
    assert done_chunks == chunks
    for r in range(n):
        if is_rs:
            want = sum(send[p][r * count:(r + 1) * count].astype(np.int64) for p in range(n)).astype(np.int32)
            assert (hits[r] == 1).all()
        else:
            want = sum(send[p].astype(np.int64) for p in range(n)).astype(np.int32)
            assert (hits[r].view(np.uint8) == 1).all()
        assert (out[r] == want).all(), (n, lanes, count, kind)
    return chunks


def test_all_reduce_and_reduce_scatter_arithmetic():
    rng = np.random.default_rng(2)
    py = random.Random(2)
    multi = 0
    for _ in range(150):
        n, lanes = py.choice([1, 2, 3, 4, 8]), py.randint(1, 7)
        stage_bytes = 1 << py.choice([10, 11, 12])
        kind = py.choice(["ar", "rs"])
        count = py.randint(1, 5 * stage_bytes // (4 * (n if kind == "rs" else 1)) + 3)
        multi += emulate_reduce(n, lanes, count, stage_bytes, kind, rng) > 1
    assert multi > 40                                      # the sizes really exercise the chunk loop


def emulate_all_gather(n, lanes, nbytes, stage_bytes, rng):
    cap, chunks = host_chunking(nbytes, stage_bytes)
    per_lane = ceil_div(ceil_div(cap, U), lanes)
    send = [rng.integers(0, 256, size=nbytes).astype(np.uint8) for _ in range(n)]
    stage = [np.zeros((2, stage_bytes + 64), dtype=np.uint8) for _ in range(n)]
    out = [np.zeros(n * nbytes, dtype=np.uint8) for _ in range(n)]
    hits = [np.zeros(n * nbytes, dtype=np.uint8) for _ in range(n)]
    half, off, done = 0, 0, 0
    while off < nbytes:
        cb = min(cap, nbytes - off)
        parts = []
        for b in range(lanes):
            lo, hi = lane_range(ceil_div(cb, U), per_lane, b)
            parts.append((lo * U, (min(hi * U, cb) - lo * U) if lo < hi else 0))
        for r in range(n):
            for bo, nb in parts:
                stage[r][half, bo:bo + nb] = send[r][off + bo:off + bo + nb]
        for r in range(n):
            for bo, nb in parts:
                for p in range(n):
                    src = send[r][off + bo:off + bo + nb] if p == r else stage[p][half, bo:bo + nb]
                    out[r][p * nbytes + off + bo:p * nbytes + off + bo + nb] = src
                    hits[r][p * nbytes + off + bo:p * nbytes + off + bo + nb] += 1
        off += cap
        half ^= 1
        done += 1
    assert done == chunks
    want = np.concatenate(send)
    for r in range(n):
        assert (hits[r] == 1).all() and (out[r] == want).all()


def test_all_gather_arithmetic():
    rng = np.random.default_rng(4)
    py = random.Random(4)
    for _ in range(120):
        n, lanes = py.choice([2, 3, 4, 8]), py.randint(1, 7)
        stage_bytes = 1 << py.choice([9, 10, 11])
        emulate_all_gather(n, lanes, py.randint(1, 5 * stage_bytes + 5), stage_bytes, rng)
