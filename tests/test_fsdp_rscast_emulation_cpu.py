"""Sequential emulation of the fused reduce-scatter + cast kernel's index arithmetic
(csrc/fused/fsdp_kernels.cu: equalised chunks on the host, staging layout, lane ranges from the
chunk capacity, the chunk loop and the ragged tail) against a numpy reduction: every output element
must be written exactly once and hold the sum over ranks. Concurrency is the business of
tests/test_protocol_model_cpu.py; this file checks that the byte offsets add up."""
import random

import numpy as np


def run(n, B, count, stageBytes):
    total = count * 2
    fullCap = (stageBytes // n) & ~15
    bytes_ = total
    capMax = fullCap
    k = (bytes_ + capMax - 1) // capMax
    cap = (((bytes_ + k - 1) // k) + 15) & ~15
    cap = min(cap, capMax)
    chunkBytes = cap
    cap_k = chunkBytes if (chunkBytes and chunkBytes < fullCap) else fullCap
    assert cap_k == cap
    perLane = (((cap + 15) >> 4) + B - 1) // B
    rng = np.random.default_rng(n * 1000 + B * 10 + count)
    send = [rng.integers(-4, 5, size=n * count).astype(np.int16) for _ in range(n)]   # stand-in for bf16 (2 bytes)
    stage = [np.zeros((2, stageBytes), dtype=np.uint8) for _ in range(n)]
    out = [np.full(count, 12345, dtype=np.int64) for _ in range(n)]
    written = [np.zeros(count, dtype=np.int32) for _ in range(n)]
    half = 0
    off = 0
    chunks = 0
    while off < total:
        cb = min(cap, total - off)
        U = (cb + 15) >> 4
        # copy-in: all ranks, all lanes
        for r in range(n):
            sb = send[r].view(np.uint8)
            for b in range(B):
                lo = min(b * perLane, U); hi = min(lo + perLane, U)
                nb = (min(hi << 4, cb) - (lo << 4)) if lo < hi else 0
                for i in range(n):
                    s = (r + i) % n
                    if nb:
                        d0 = s * cap + (lo << 4)
                        s0 = s * total + off + (lo << 4)
                        assert d0 + nb <= stageBytes
                        stage[r][half, d0:d0 + nb] = sb[s0:s0 + nb]
        # reduce
        for r in range(n):
            stOff = r * cap
            outElems = cb // 2
            for b in range(B):
                lo = min(b * perLane, U); hi = min(lo + perLane, U)
                for u in range(lo, hi):
                    acc = np.zeros(8, dtype=np.int64)
                    for p in range(n):
                        v = stage[p][half, stOff + (u << 4): stOff + (u << 4) + 16].view(np.int16)
                        acc += v
                    e0 = u * 8
                    for kk in range(8):
                        if e0 + kk < outElems:
                            out[r][off // 2 + e0 + kk] = acc[kk]
                            written[r][off // 2 + e0 + kk] += 1
        off += cap; half ^= 1; chunks += 1
    assert chunks == (bytes_ + cap - 1) // cap
    for r in range(n):
        want = sum(send[p][r * count:(r + 1) * count].astype(np.int64) for p in range(n))
        assert (written[r] == 1).all(), (n, B, count, "coverage")
        assert (out[r] == want).all(), (n, B, count)


def test_index_arithmetic_matches_numpy_over_random_shapes():
    rng = random.Random(1)
    for _ in range(120):
        n = rng.choice([2, 4, 8])
        lanes = rng.randint(1, 9)
        stage_bytes = 1 << rng.choice([12, 13, 14])
        count = rng.randint(1, 5 * stage_bytes // (2 * n) + 7)
        run(n, lanes, count, stage_bytes)


def test_single_chunk_messages_use_every_lane():
    # a message far smaller than the staging share still spreads over the lanes (the chunk capacity is the message itself)
    run(8, 6, 50, 1 << 14)
    run(2, 9, 8, 1 << 12)
