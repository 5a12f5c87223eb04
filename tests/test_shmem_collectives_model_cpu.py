"""The data movement of the device-initiated layer's block collectives (csrc/include/b200coll/shmem_device.cuh) restated
on numpy arrays, one array per PE, with the PEs' steps interleaved in arbitrary order inside each barrier-delimited phase:
the two-step reduction must be right in place for every order (each slice is folded only by its owner, fetched only after
the barrier), while a one-step "everyone folds everything in place" is shown to depend on the order; broadcast, fcollect
and alltoall must land every block where OpenSHMEM says."""
import itertools

import numpy as np


def _slices(n, count):
    per = -(-count // n)
    return [(min(count, per * p), min(count, per * p + per)) for p in range(n)]


def two_step_reduce(src, dst, order1, order2):
    """src / dst: lists of arrays (dst[p] may be src[p]). order1 / order2: the order in which PEs run step 1 / step 2."""
    n, count = len(src), len(src[0])
    sl = _slices(n, count)
    for p in order1:                      # step 1: PE p folds slice p of every PE's source into its own dest
        lo, hi = sl[p]
        acc = src[0][lo:hi].copy()
        for q in range(1, n):
            acc = acc + src[q][lo:hi]
        dst[p][lo:hi] = acc
    for p in order2:                      # step 2 (after the barrier): PE p fetches the other slices from their owners
        for k in range(1, n):
            q = (p + k) % n
            lo, hi = sl[q]
            dst[p][lo:hi] = dst[q][lo:hi]


def one_step_reduce_in_place(buf, order):
    n = len(buf)
    for p in order:
        acc = buf[0].copy()
        for q in range(1, n):
            acc = acc + buf[q]
        buf[p][:] = acc


def test_two_step_reduction_is_right_in_place_for_every_order_of_the_pes():
    n, count = 3, 10                                                      # 10 elements over 3 PEs: slices 4, 4, 2
    want = sum(np.arange(count) * (p + 1) + p for p in range(n))
    for o1 in itertools.permutations(range(n)):
        for o2 in itertools.permutations(range(n)):
            buf = [np.arange(count) * (p + 1) + p for p in range(n)]
            two_step_reduce(buf, buf, o1, o2)                              # dest is source
            assert all(np.array_equal(b, want) for b in buf), (o1, o2)
    src = [np.arange(5) + p for p in range(4)]                             # more PEs than whole slices: some are empty or short
    dst = [np.zeros(5, dtype=src[0].dtype) for _ in range(4)]
    two_step_reduce(src, dst, range(4), reversed(range(4)))
    assert all(np.array_equal(d, 4 * np.arange(5) + 6) for d in dst) and np.array_equal(src[2], np.arange(5) + 2)
    assert _slices(4, 5) == [(0, 2), (2, 4), (4, 5), (5, 5)]


def test_one_step_in_place_reduction_depends_on_the_order():
    """Why the reduction is not a plain 'read everybody, write my own': the first PE to finish changes what the others read."""
    n, count = 3, 4
    want = sum(np.full(count, p + 1) for p in range(n))
    buf = [np.full(count, p + 1) for p in range(n)]
    one_step_reduce_in_place(buf, range(n))
    assert np.array_equal(buf[0], want) and not np.array_equal(buf[1], want)


def test_push_collectives_place_every_block():
    n, cnt = 4, 3
    src = [np.arange(cnt) + 100 * p for p in range(n)]
    # fcollect: PE p writes its block into dest[p] of every PE
    dest = [np.zeros((n, cnt), dtype=int) for _ in range(n)]
    for p in range(n):
        for i in range(n):
            dest[(p + i) % n][p] = src[p]
    assert all(np.array_equal(d, np.stack(src)) for d in dest)
    # alltoall: block q of PE p's source becomes block p of PE q's dest
    a = [np.array([[1000 * p + 10 * q + j for j in range(cnt)] for q in range(n)]) for p in range(n)]
    dest = [np.zeros((n, cnt), dtype=int) for _ in range(n)]
    for p in range(n):
        for i in range(n):
            q = (p + i) % n
            dest[q][p] = a[p][q]
    for q in range(n):
        assert np.array_equal(dest[q], np.array([[1000 * p + 10 * q + j for j in range(cnt)] for p in range(n)]))
    # broadcast from root 1
    dest = [np.zeros(cnt, dtype=int) for _ in range(n)]
    for i in range(n):
        dest[(1 + i) % n][:] = src[1]
    assert all(np.array_equal(d, src[1]) for d in dest)


def test_team_pe_translation_matches_the_set_definition():
    """b200shmem_team_translate_pe (host form; the device form is the same arithmetic) against the definition: member idx of
    src is PE start + idx * stride; its number in dst is its position in dst's member list, or -1."""
    import ctypes

    from rocm_systems_b200 import shmem

    lib = shmem._l()
    teams = [(0, 1, 8), (0, 2, 4), (1, 2, 4), (0, 4, 2), (2, 3, 2), (5, 1, 3), (7, 1, 1)]
    for s in teams:
        for d in teams:
            src, dst = shmem.Team(*s, 0, None, None), shmem.Team(*d, 0, None, None)
            for idx in range(-1, s[2] + 1):
                got = lib.b200shmem_team_translate_pe(ctypes.byref(src), idx, ctypes.byref(dst))
                if 0 <= idx < s[2]:
                    pe = s[0] + idx * s[1]
                    want = dst.pes().index(pe) if pe in dst.pes() else -1
                else:
                    want = -1
                assert got == want, (s, d, idx, got, want)
