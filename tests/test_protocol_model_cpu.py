"""A model check of the staged, software-pipelined collective protocol on the CPU.

Every (rank, lane) of a launch is a process; the only synchronisation is the per-lane barrier
between the same lane of all ranks, plus program order inside a thread group. The model lists
every staging access of a launch — who, in which barrier epoch, which bytes of whose staging half,
read or write — with the same geometry the kernels use (csrc/coll/kernels.cuh: slice stride and
lane ranges derived from the chunk capacity only), and then looks for pairs of accesses that touch
the same bytes, at least one writing, with nothing ordering them. It has to find none for the
committed geometry at any message size, and it has to find the overlap of the geometry that
derived lane ranges from each chunk's own size (a short last chunk then lands in other lanes'
ranges), which is the data race large messages once hit.
"""
import itertools
import random

import pytest

U = 16  # bytes per unit


def ceil_div(a, b):
    return (a + b - 1) // b


class Geometry:
    """Where chunk data lives in a staging half and which lane handles it."""

    def __init__(self, n, lanes, total, cap, kind, by_capacity=True):
        self.n, self.B, self.total, self.cap, self.kind, self.by_capacity = n, lanes, total, cap, kind, by_capacity
        cap_units = ceil_div(cap, U)
        self.su_full = cap_units if kind == "rs" else ceil_div(cap_units, n)

    def chunk_bytes(self, k):
        off = k * self.cap
        return min(self.cap, self.total - off)

    def chunks(self):
        return ceil_div(self.total, self.cap)

    def su(self, k):
        if self.by_capacity:
            return self.su_full
        units = ceil_div(self.chunk_bytes(k), U)      # the geometry that follows each chunk's own size
        return units if self.kind == "rs" else ceil_div(units, self.n)

    def slice_bytes(self, k, s):
        cb = self.chunk_bytes(k)
        if self.kind == "rs":
            return cb
        lo = s * self.su(k) * U
        return max(0, min(cb - lo, self.su(k) * U))

    def slice_stage(self, k, s):
        return s * self.cap if self.kind == "rs" else s * self.su(k) * U

    def lane_range(self, k, s, b):
        """Byte range [lo, hi) inside the staging half that lane b handles of slice s of chunk k."""
        sb = self.slice_bytes(k, s)
        units = ceil_div(sb, U)
        if self.by_capacity:
            per = ceil_div(self.su_full, self.B)
        else:
            per = ceil_div(units, self.B) if units else 0
        lo = min(b * per, units)
        hi = min(lo + per, units)
        base = self.slice_stage(k, s)
        return base + lo * U, base + hi * U


def accesses(g: Geometry, half0: int = 0):
    """All staging accesses of one launch of the pipelined staged reduce (all-reduce or
    reduce-scatter): tuples (rank, lane, group, epoch, target_rank, half, lo, hi, is_write).
    ``half0`` is the staging half of the launch's first chunk."""
    out = []
    K = g.chunks()
    has_out = g.kind == "ar"
    for r, b in itertools.product(range(g.n), range(g.B)):
        def copy(k, epoch, write, group):
            for s in range(g.n):
                lo, hi = g.lane_range(k, s, b)
                if lo < hi:
                    out.append((r, b, group, epoch, r, (k + half0) & 1, lo, hi, write))
        copy(0, 0, True, "all")                                   # prologue: copy-in of chunk 0, then barrier
        for k in range(K):
            epoch = k + 1
            more, prev_out = k + 1 < K, has_out and k > 0
            split = more or prev_out
            lo, hi = g.lane_range(k, r, b)                        # this rank reduces slice r
            if lo < hi:
                for p in range(g.n):
                    out.append((r, b, "reduce" if split else "all", epoch, p, (k + half0) & 1, lo, hi, False))
                    if has_out:
                        out.append((r, b, "reduce" if split else "all", epoch, p, (k + half0) & 1, lo, hi, True))
            if prev_out:
                copy(k - 1, epoch, False, "copy")                 # copy-out of the previous chunk ...
            if more:
                copy(k + 1, epoch, True, "copy")                  # ... then (group barrier) copy-in of the next
        if has_out:
            copy(K - 1, K + 1, False, "all")                      # epilogue after the last barrier
    return out


def races(acc):
    """Pairs of conflicting accesses that nothing orders."""
    by_target = {}
    for a in acc:
        by_target.setdefault((a[4], a[5]), []).append(a)
    found = []
    for items in by_target.values():
        items.sort(key=lambda a: a[6])
        for i, a in enumerate(items):
            for c in items[i + 1:]:
                if c[6] >= a[7]:
                    break                                          # sorted by start: no later item overlaps a
                if not (a[8] or c[8]):
                    continue                                       # two reads
                same_proc = a[0] == c[0] and a[1] == c[1]
                if a[1] == c[1] and a[3] != c[3]:
                    continue                                       # same lane, a barrier in between
                if same_proc and (a[2] == c[2] or "all" in (a[2], c[2])):
                    continue                                       # program order within a thread group
                found.append((a, c))
    return found


CASES = [
    # n, lanes, total bytes, chunk capacity, kind
    (2, 4, 5 * 4096 + 1520, 4096, "ar"),     # short last chunk
    (4, 6, 7 * 8192 + 48, 8192, "ar"),
    (8, 5, 3 * 16384 + 16, 16384, "ar"),
    (2, 4, 4 * 4096, 4096, "ar"),            # equal chunks
    (4, 3, 9 * 2048 + 700, 2048, "rs"),
    (8, 7, 2 * 4096 + 4000, 4096, "rs"),
    (3, 4, 1000, 4096, "ar"),                # single chunk
]


@pytest.mark.parametrize("n,lanes,total,cap,kind", CASES)
def test_committed_geometry_has_no_unordered_conflicts(n, lanes, total, cap, kind):
    g = Geometry(n, lanes, total, cap, kind, by_capacity=True)
    assert races(accesses(g)) == []
    # and every byte of every chunk is handled by exactly one lane
    for k in range(g.chunks()):
        for s in range(n):
            covered = sorted(g.lane_range(k, s, b) for b in range(lanes))
            covered = [c for c in covered if c[0] < c[1]]
            sb = g.slice_bytes(k, s)
            if sb == 0:
                assert covered == []
                continue
            assert covered[0][0] == g.slice_stage(k, s) and covered[-1][1] == g.slice_stage(k, s) + ceil_div(sb, U) * U
            assert all(a[1] == b_[0] for a, b_ in zip(covered, covered[1:]))


def test_random_sizes_are_race_free():
    rng = random.Random(7)
    for _ in range(60):
        n = rng.choice([2, 3, 4, 8])
        lanes = rng.randint(1, 6)
        cap = U * rng.randint(n, 300)
        total = rng.randint(1, 6 * cap)
        kind = rng.choice(["ar", "rs"])
        g = Geometry(n, lanes, total, cap, kind, by_capacity=True)
        assert races(accesses(g)) == [], (n, lanes, total, cap, kind)


def test_chunk_sized_geometry_is_caught():
    """Lane ranges that follow each chunk's own size: the copy-in of a short last chunk by one lane
    overlaps what another lane still copies out of the same half."""
    g = Geometry(2, 4, 5 * 4096 + 1520, 4096, "ar", by_capacity=False)
    bad = races(accesses(g))
    assert bad, "the model no longer sees the cross-lane overlap"
    a, c = bad[0]
    assert a[1] != c[1] and (a[8] or c[8])                         # different lanes, one of them writing
    # with equal chunks the two geometries coincide and nothing is wrong
    assert races(accesses(Geometry(2, 4, 4 * 4096, 4096, "ar", by_capacity=False))) == []


def last_epoch(g: Geometry) -> int:
    """Epoch of the accesses after the launch's last barrier (all-reduce: the epilogue copy-out;
    reduce-scatter: the last chunk's reduce, which no barrier follows)."""
    return g.chunks() + 1 if g.kind == "ar" else g.chunks()


def cross_call_races(ga: Geometry, gb: Geometry):
    """Launch A then launch B on every rank's stream, B starting on the half after A's last chunk.
    A rank's own launches are ordered by its stream; across ranks an access of A is ordered before an
    access of B if a barrier follows it in A (every rank takes part in every lane's barriers and
    finishes A before it starts B) or a barrier precedes the other in B. What is left unordered is
    A's accesses after its last barrier against B's prologue, on different ranks."""
    a_tail = [x for x in accesses(ga, 0) if x[3] == last_epoch(ga)]
    b_head = [y for y in accesses(gb, ga.chunks() & 1) if y[3] == 0]
    found = []
    for x in a_tail:
        for y in b_head:
            if x[0] != y[0] and x[4] == y[4] and x[5] == y[5] and x[6] < y[7] and y[6] < x[7] and (x[8] or y[8]):
                found.append((x, y))
    return found


def test_back_to_back_launches_need_no_trailing_barrier():
    rng = random.Random(11)
    for _ in range(40):
        n = rng.choice([2, 4, 8])
        cap = U * rng.randint(n, 200)
        ga = Geometry(n, rng.randint(1, 5), rng.randint(1, 5 * cap), cap, rng.choice(["ar", "rs"]))
        capb = U * rng.randint(n, 200)
        gb = Geometry(n, rng.randint(1, 5), rng.randint(1, 5 * capb), capb, rng.choice(["ar", "rs"]))   # other size, other lane count
        assert cross_call_races(ga, gb) == []
    # the invariant is the alternation of halves: start B on the half A just used and a reduce-scatter's
    # last peer reads meet the next launch's copy-in
    ga = Geometry(2, 2, 3 * 1024, 1024, "rs")
    gb = Geometry(2, 2, 1024, 1024, "rs")
    a_tail = [x for x in accesses(ga, 0) if x[3] == last_epoch(ga)]
    b_head_wrong = [y for y in accesses(gb, (ga.chunks() - 1) & 1) if y[3] == 0]
    assert any(x[0] != y[0] and x[4] == y[4] and x[5] == y[5] and x[6] < y[7] and y[6] < x[7] and (x[8] or y[8]) for x in a_tail for y in b_head_wrong)


# ---- the pipelined all-gather (kStagedCopy): staging holds the rank's own contribution only ----
def ag_part(total, cap, lanes, k, b, by_capacity=True):
    cb = min(cap, total - k * cap)
    units = ceil_div(cb, U)
    per = ceil_div(ceil_div(cap, U), lanes) if by_capacity else (ceil_div(units, lanes) if units else 0)
    lo = min(b * per, units)
    hi = min(lo + per, units)
    return lo * U, hi * U


def ag_accesses(n, lanes, total, cap, by_capacity=True):
    out = []
    K = ceil_div(total, cap)
    for r, b in itertools.product(range(n), range(lanes)):
        lo, hi = ag_part(total, cap, lanes, 0, b, by_capacity)
        if lo < hi:
            out.append((r, b, "all", 0, r, 0, lo, hi, True))                    # prologue: stage chunk 0
        for k in range(K):
            epoch, more = k + 1, k + 1 < K
            lo, hi = ag_part(total, cap, lanes, k, b, by_capacity)
            if lo < hi:
                for p in range(n):
                    if p != r:
                        out.append((r, b, "pull", epoch, p, k & 1, lo, hi, False))   # read the peers' staging
            if more:
                lo, hi = ag_part(total, cap, lanes, k + 1, b, by_capacity)
                if lo < hi:
                    out.append((r, b, "copy", epoch, r, (k + 1) & 1, lo, hi, True))  # stage the next chunk meanwhile
    return out


def test_pipelined_all_gather_is_race_free_and_the_old_split_is_not():
    rng = random.Random(3)
    for _ in range(60):
        n, lanes = rng.choice([2, 3, 4, 8]), rng.randint(1, 6)
        cap = U * rng.randint(4, 200)
        total = rng.randint(1, 6 * cap)
        assert races(ag_accesses(n, lanes, total, cap)) == [], (n, lanes, total, cap)
    # ranges that follow the chunk's own size: a short last chunk staged by one lane overlaps what a
    # remote rank's other lane still pulls of the chunk before last
    assert races(ag_accesses(2, 4, 5 * 4096 + 1520, 4096, by_capacity=False))


# ---- the fused reduce-scatter + cast of the FSDP path: same staging, no software pipeline ----
def rs_cast_accesses(g: Geometry):
    """copy-in(k) | barrier | reduce(k) | copy-in(k+1) | barrier | ... : one barrier per chunk, the next
    copy-in follows the reduce without one."""
    out = []
    for r, b in itertools.product(range(g.n), range(g.B)):
        epoch = 0
        for k in range(g.chunks()):
            for s in range(g.n):
                lo, hi = g.lane_range(k, s, b)
                if lo < hi:
                    out.append((r, b, "all", epoch, r, k & 1, lo, hi, True))
            epoch += 1                                                     # the barrier
            lo, hi = g.lane_range(k, r, b)
            if lo < hi:
                for p in range(g.n):
                    out.append((r, b, "all", epoch, p, k & 1, lo, hi, False))
    return out


def test_fused_reduce_scatter_cast_geometry():
    rng = random.Random(5)
    for _ in range(60):
        n, lanes = rng.choice([2, 4, 8]), rng.randint(1, 6)
        cap = U * rng.randint(2, 200)
        g = Geometry(n, lanes, rng.randint(1, 7 * cap), cap, "rs", by_capacity=True)
        assert races(rs_cast_accesses(g)) == [], (n, lanes, g.total, cap)
    # lane ranges cut from each chunk's own size: the short last chunk's copy-in crosses into ranges
    # that another lane of a peer may still be reading from two chunks earlier
    assert races(rs_cast_accesses(Geometry(2, 4, 6 * 4096 + 1520, 4096, "rs", by_capacity=False)))


# ---- the scatter-and-forward broadcast (kStagedCopy, three ranks and more, peer stores only) ----
def bc_region(part_lo, part_hi, lane_cap_bytes, m, o, by_capacity=True):
    """Region o of the m regions a lane's part [part_lo, part_hi) of a chunk is cut into."""
    nbytes = part_hi - part_lo
    basis = lane_cap_bytes if by_capacity else nbytes
    sub = ceil_div(ceil_div(basis, m), U) * U if basis else 0
    lo = min(o * sub, nbytes)
    hi = min(lo + sub, nbytes)
    return part_lo + lo, part_lo + hi


def bc_accesses(n, lanes, total, cap, root, by_capacity=True, half0=0):
    out = []
    K = ceil_div(total, cap)
    m = n - 1
    lane_cap = ceil_div(ceil_div(cap, U), lanes) * U
    owner = lambda o: (root + 1 + o) % n
    own = lambda r: (r - root - 1 + n) % n

    def regions(k, b):
        lo, hi = ag_part(total, cap, lanes, k, b)          # lane parts follow the capacity (as in the all-gather)
        return [bc_region(lo, hi, lane_cap, m, o, by_capacity) for o in range(m)]

    for b in range(lanes):
        for o, (lo, hi) in enumerate(regions(0, b)):       # prologue: the root stores chunk 0, region o into its owner
            if lo < hi:
                out.append((root, b, "all", 0, owner(o), half0, lo, hi, True))
        for k in range(K):
            epoch, half, more = k + 1, (half0 + k) & 1, k + 1 < K
            if more:
                for o, (lo, hi) in enumerate(regions(k + 1, b)):
                    if lo < hi:
                        out.append((root, b, "push", epoch, owner(o), half ^ 1, lo, hi, True))
            for r in range(n):
                if r == root:
                    continue
                lo, hi = regions(k, b)[own(r)]
                if lo < hi:
                    out.append((r, b, "fwd", epoch, r, half, lo, hi, False))                  # read the region the root left here
                    for p in range(n):
                        if p not in (r, root):
                            out.append((r, b, "fwd", epoch, p, half, lo, hi, True))          # forward it
                    out.append((r, b, "out", epoch, r, half, lo, hi, False))                  # copy it to recv
                if k > 0:
                    for o, (qlo, qhi) in enumerate(regions(k - 1, b)):
                        if o != own(r) and qlo < qhi:
                            out.append((r, b, "out", epoch, r, half ^ 1, qlo, qhi, False))    # forwarded regions of the chunk before
        for r in range(n):                                                                    # behind the last barrier
            if r == root:
                continue
            for o, (qlo, qhi) in enumerate(regions(K - 1, b)):
                if o != own(r) and qlo < qhi:
                    out.append((r, b, "all", K + 1, r, (half0 + K - 1) & 1, qlo, qhi, False))
    return out


def test_scatter_and_forward_broadcast_is_race_free_and_chunk_sized_regions_are_not():
    rng = random.Random(7)
    for _ in range(80):
        n, lanes = rng.choice([3, 4, 5, 8]), rng.randint(1, 5)
        cap = U * rng.randint(6, 240)
        total = rng.randint(1, 7 * cap)
        root = rng.randrange(n)
        assert races(bc_accesses(n, lanes, total, cap, root, half0=rng.randint(0, 1))) == [], (n, lanes, total, cap, root)
    # regions cut from each chunk's own size: the root's stores of a short chunk k + 1 land on regions of chunk k - 1
    # (same half) that their receivers are still copying out
    assert races(bc_accesses(4, 4, 4 * 838880 + 838816, 838880, 1, by_capacity=False))


# ---- the staged all-to-all: one slot per source rank in a staging half, push step k + 1 while step k is copied out ----
def a2a_accesses(n, lanes, total, stage_bytes, half0=0):
    out = []
    slot = (stage_bytes // n) // U * U
    cap = min(slot, ceil_div(total, U) * U)
    K = ceil_div(total, cap)
    for r, b in itertools.product(range(n), range(lanes)):
        lo, hi = ag_part(total, cap, lanes, 0, b)
        for p in range(n):
            if p != r and lo < hi:
                out.append((r, b, "all", 0, p, half0, r * slot + lo, r * slot + hi, True))
        for k in range(K):
            epoch, half, more = k + 1, (half0 + k) & 1, k + 1 < K
            if more:
                lo, hi = ag_part(total, cap, lanes, k + 1, b)
                for p in range(n):
                    if p != r and lo < hi:
                        out.append((r, b, "push", epoch, p, half ^ 1, r * slot + lo, r * slot + hi, True))
            lo, hi = ag_part(total, cap, lanes, k, b)
            for s in range(n):
                if s != r and lo < hi:
                    out.append((r, b, "out" if more else "all", epoch, r, half, s * slot + lo, s * slot + hi, False))
    return out


def test_staged_all_to_all_is_race_free():
    rng = random.Random(9)
    for _ in range(80):
        n, lanes = rng.choice([2, 3, 4, 8]), rng.randint(1, 5)
        stage = U * n * rng.randint(8, 200)
        total = rng.randint(1, 6 * (stage // n))
        assert races(a2a_accesses(n, lanes, total, stage, half0=rng.randint(0, 1))) == [], (n, lanes, total, stage)
