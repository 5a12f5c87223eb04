"""Exhaustive interleaving checks of the two flag protocols that are not barrier-based
(csrc/coll/kernels.cuh): the send/recv FIFO with credits (kP2p) and the flag-in-data all-reduce (kLLAllReduce).

Each rank is a small state machine whose steps are the protocol's individually atomic memory operations
(a wait that is satisfied, one piece of a slot copy, a release store of a counter, one 16-byte line store).
Every reachable interleaving is explored. A run must never read a slot or a line that does not hold exactly
the message it expects, and must never get stuck before every rank has finished. The same explorer has to find a
counterexample in broken variants of each protocol (no credit wait, counter published before the data, a single
line buffer), which shows that it can."""
from collections import deque


def explore(initial, step, done, nprocs, limit=2_000_000):
    """Breadth-first search over all interleavings. ``step(state, pid)`` returns the next state, None when pid cannot
    move (blocked or finished), or raises AssertionError on a safety violation. Returns (states, deadlocks)."""
    seen = {initial}
    queue = deque([initial])
    deadlocks = 0
    while queue:
        s = queue.popleft()
        moved = False
        for pid in range(nprocs):
            t = step(s, pid)
            if t is None:
                continue
            moved = True
            if t not in seen:
                seen.add(t)
                assert len(seen) < limit, "state space larger than expected"
                queue.append(t)
        if not moved and not done(s):
            deadlocks += 1
    return len(seen), deadlocks


# ---- FIFO with credits ---------------------------------------------------------------------------------------------
# State: (s_pc, sent, r_pc, recvd, tail, head, slots) with slots a tuple of (first half, second half) message ids.
def fifo_model(nslots, nmsgs, wait_credit=True, publish_after_write=True):
    def step(st, pid):
        s_pc, sent, r_pc, recvd, tail, head, slots = st
        if pid == 0:  # sender
            if sent == nmsgs:
                return None
            slot = sent % nslots
            if s_pc == 0:  # waitGe64(head, sent + 1 - slots)
                if wait_credit and head < sent + 1 - nslots:
                    return None
                if not publish_after_write:  # broken variant: the tail moves before the data is there
                    return (1, sent, r_pc, recvd, sent + 1, head, slots)
                return (1, sent, r_pc, recvd, tail, head, slots)
            if s_pc in (1, 2):  # the copy into the slot, in two pieces
                a, b = slots[slot]
                piece = (sent, b) if s_pc == 1 else (a, sent)
                return (s_pc + 1, sent, r_pc, recvd, tail, head, slots[:slot] + (piece,) + slots[slot + 1:])
            return (0, sent + 1, r_pc, recvd, max(tail, sent + 1), head, slots)  # fence + release store of the tail
        if recvd == nmsgs:  # receiver
            return None
        slot = recvd % nslots
        if r_pc == 0:  # waitGe64(tail, recvd + 1)
            return (s_pc, sent, 1, recvd, tail, head, slots) if tail >= recvd + 1 else None
        if r_pc in (1, 2):  # the copy out of the slot, in two pieces
            got = slots[slot][r_pc - 1]
            assert got == recvd, f"message {recvd}: read piece {r_pc} of slot {slot} holding {got}"
            return (s_pc, sent, r_pc + 1, recvd, tail, head, slots)
        return (s_pc, sent, 0, recvd + 1, tail, recvd + 1, slots)  # release store of the head

    initial = (0, 0, 0, 0, 0, 0, tuple((-1, -1) for _ in range(nslots)))
    return initial, step, (lambda st: st[1] == nmsgs and st[3] == nmsgs)


def test_fifo_with_credits_delivers_every_message_in_every_interleaving():
    for nslots, nmsgs in [(1, 4), (2, 7), (4, 11)]:
        initial, step, done = fifo_model(nslots, nmsgs)
        states, deadlocks = explore(initial, step, done, 2)
        assert deadlocks == 0 and states > nmsgs * 8


def _violates(initial, step, done, nprocs):
    try:
        _, deadlocks = explore(initial, step, done, nprocs)
    except AssertionError:
        return True
    return deadlocks > 0


def test_fifo_checker_finds_the_bugs_it_is_meant_to_find():
    assert _violates(*fifo_model(2, 5, wait_credit=False), 2)            # a slot is overwritten before it was read
    assert _violates(*fifo_model(2, 5, publish_after_write=False), 2)    # the receiver is told before the data is there


# ---- flag-in-data all-reduce -----------------------------------------------------------------------------------------
# Per rank: call number k (1-based), phase ("send", next peer index) or ("recv", next peer index); memory:
# line[dst][buf][src] = (data, flag) written in one store. Data of rank r in call k is (r, k).
def ll_model(n, ncalls, nbufs=2):
    peers = [[(r + d) % n for d in range(1, n)] for r in range(n)]

    def step(st, pid):
        procs, mem = st
        k, phase, idx = procs[pid]
        if k > ncalls:
            return None
        buf = k % nbufs
        if phase == 0:  # one 16-byte line {data, flag} into the next peer
            dst = peers[pid][idx]
            cell = (dst * nbufs + buf) * n + pid
            mem2 = mem[:cell] + (((pid, k), k),) + mem[cell + 1:]
            nxt = (k, 0, idx + 1) if idx + 1 < n - 1 else (k, 1, 0)
            return (procs[:pid] + (nxt,) + procs[pid + 1:], mem2)
        src = peers[pid][idx]  # spin on the line of the next source
        data, flag = mem[(pid * nbufs + buf) * n + src]
        if flag != k:
            return None
        assert data == (src, k), f"rank {pid} call {k}: line of {src} holds {data}"
        nxt = (k, 1, idx + 1) if idx + 1 < n - 1 else (k + 1, 0, 0)
        return (procs[:pid] + (nxt,) + procs[pid + 1:], mem)

    initial = (tuple((1, 0, 0) for _ in range(n)), tuple(((None, None), 0) for _ in range(n * nbufs * n)))
    return initial, step, (lambda st: all(p[0] > ncalls for p in st[0]))


def test_ll_all_reduce_with_two_alternating_buffers_never_loses_a_line():
    for n, ncalls in [(2, 6), (3, 4)]:
        initial, step, done = ll_model(n, ncalls)
        states, deadlocks = explore(initial, step, done, n)
        assert deadlocks == 0 and states > 3 * n * ncalls


def test_ll_checker_finds_the_single_buffer_overwrite():
    # With one buffer a rank that is a call ahead overwrites a line its peer has not consumed; the peer then waits for a
    # flag value that is gone.
    assert _violates(*ll_model(2, 3, nbufs=1), 2)
    assert _violates(*ll_model(3, 3, nbufs=1), 3)


def test_ll_all_reduce_four_ranks():
    initial, step, done = ll_model(4, 2)
    states, deadlocks = explore(initial, step, done, 4)
    assert deadlocks == 0 and states > 1000


# ---- the lane barrier -----------------------------------------------------------------------------------------------
# ctaBarrier: epoch += 1; store the epoch into slot [rank] of every peer (release); wait until every slot of the own
# workspace has reached the epoch (acquire). Between barriers a rank does one unit of "work" on a shared counter that
# lets the model see whether anybody ran ahead: work of round k may start only after every rank finished round k - 1.
def barrier_model(n, rounds, compare_ge=True):
    def step(st, pid):
        procs, slots, work = st
        k, pc, idx = procs[pid]          # round (1-based), 0 = work, 1 = stores, 2 = waits
        if k > rounds:
            return None
        if pc == 0:
            assert all(w >= k - 1 for w in work), f"rank {pid} started round {k} while a peer had not finished round {k - 1}: {work}"
            work2 = work[:pid] + (k,) + work[pid + 1:]
            return (procs[:pid] + ((k, 1, 0),) + procs[pid + 1:], slots, work2)
        if pc == 1:  # one release store per peer, own slot included
            cell = idx * n + pid
            slots2 = slots[:cell] + (k,) + slots[cell + 1:]
            nxt = (k, 1, idx + 1) if idx + 1 < n else (k, 2, 0)
            return (procs[:pid] + (nxt,) + procs[pid + 1:], slots2, work)
        seen = slots[pid * n + idx]
        if (seen < k) if compare_ge else (seen != k):
            return None
        nxt = (k, 2, idx + 1) if idx + 1 < n else (k + 1, 0, 0)
        return (procs[:pid] + (nxt,) + procs[pid + 1:], slots, work)

    initial = (tuple((1, 0, 0) for _ in range(n)), tuple(0 for _ in range(n * n)), tuple(0 for _ in range(n)))
    return initial, step, (lambda st: all(p[0] > rounds for p in st[0]))


def test_lane_barrier_orders_rounds_and_never_sticks():
    for n, rounds in [(2, 5), (3, 3)]:
        initial, step, done = barrier_model(n, rounds)
        states, deadlocks = explore(initial, step, done, n)
        assert deadlocks == 0 and states > 10 * n * rounds


def test_barrier_checker_finds_the_equality_wait():
    # Waiting for "slot == epoch" instead of ">=": a fast peer may already have stored the next epoch.
    assert _violates(*barrier_model(2, 3, compare_ge=False), 2)


# ---- expert-parallel dispatch / combine across calls (csrc/fused/ep_kernels.cu) ------------------------------------
# One expert per rank, every rank sends one row to every rank (itself included) per call. Steps of a rank in call k,
# parity p = k & 1:  clear cnt[p ^ 1] locally;  per destination: reserve a row (remote atomic add on cnt[p]) and store
# the payload;  store done[p][rank] = k // 2 + 1 at every rank;  wait until every done[p][*] has reached it;  read the
# local payload rows and cnt[p] (dequantise + expert GEMM) and write the output rows;  barrier;  pull the own token's
# output row from every owner (combine). Payload and output buffers are NOT double buffered, only the counters are.
def ep_model(n, ncalls, barrier_before_combine=True):
    CLEAR, SEND, DONE, WAIT, EXPERT, BAR_IN, BAR_OUT, PULL = range(8)

    def step(st, pid):
        procs, cnt, done, payload, out, bar = st
        k, pc, idx = procs[pid]
        if k > ncalls:
            return None
        p = k & 1
        mark = k // 2 + 1

        def upd(t, i, v):
            return t[:i] + (v,) + t[i + 1:]

        def goto(npc, nidx=0, nk=None):
            return upd(procs, pid, (k if nk is None else nk, npc, nidx))

        if pc == CLEAR:
            return (goto(SEND), upd(cnt, pid * 2 + (p ^ 1), 0), done, payload, out, bar)
        if pc == SEND:  # reserve a row at rank idx and store (source, call) there
            row = cnt[idx * 2 + p]
            assert row < n, f"rank {pid} call {k}: expert of rank {idx} already holds {row} rows"
            cnt2 = upd(cnt, idx * 2 + p, row + 1)
            pay2 = upd(payload, idx * n + row, (pid, k))
            return (goto(SEND, idx + 1) if idx + 1 < n else goto(DONE), cnt2, done, pay2, out, bar)
        if pc == DONE:
            d2 = upd(done, (idx * 2 + p) * n + pid, mark)
            return (goto(DONE, idx + 1) if idx + 1 < n else goto(WAIT), cnt, d2, payload, out, bar)
        if pc == WAIT:
            if done[(pid * 2 + p) * n + idx] < mark:
                return None
            return (goto(WAIT, idx + 1) if idx + 1 < n else goto(EXPERT), cnt, done, payload, out, bar)
        if pc == EXPERT:  # every row of this call is here, nothing of another call; outputs keyed by source rank
            assert cnt[pid * 2 + p] == n, f"rank {pid} call {k}: {cnt[pid * 2 + p]} rows"
            rows = payload[pid * n:(pid + 1) * n]
            assert sorted(rows) == [(s, k) for s in range(n)], f"rank {pid} call {k}: rows {rows}"
            out2 = out
            for s, _ in rows:
                out2 = upd(out2, pid * n + s, k)
            return (goto(BAR_IN if barrier_before_combine else PULL), cnt, done, payload, out2, bar)
        if pc == BAR_IN:  # the communicator's barrier: arrive, then wait for everybody
            return (goto(BAR_OUT), cnt, done, payload, out, upd(bar, pid, bar[pid] + 1))
        if pc == BAR_OUT:
            if min(bar) < bar[pid]:
                return None
            return (goto(PULL), cnt, done, payload, out, bar)
        got = out[idx * n + pid]  # PULL: the row expert idx computed for this rank's token
        assert got == k, f"rank {pid} call {k}: pulled an output of call {got} from rank {idx}"
        return (goto(PULL, idx + 1) if idx + 1 < n else goto(CLEAR, 0, k + 1), cnt, done, payload, out, bar)

    initial = (tuple((1, CLEAR, 0) for _ in range(n)), tuple(0 for _ in range(2 * n)), tuple(0 for _ in range(2 * n * n)),
               tuple((None, 0) for _ in range(n * n)), tuple(0 for _ in range(n * n)), tuple(0 for _ in range(n)))
    return initial, step, (lambda st: all(pr[0] > ncalls for pr in st[0]))


def test_ep_dispatch_combine_is_safe_across_calls_with_single_payload_and_output_buffers():
    initial, step, done = ep_model(2, 4)
    states, deadlocks = explore(initial, step, done, 2)
    assert deadlocks == 0 and states > 200
    initial, step, done = ep_model(3, 2)
    states, deadlocks = explore(initial, step, done, 3)
    assert deadlocks == 0


def test_ep_checker_finds_the_missing_barrier():
    # Without the barrier between the expert GEMMs and the combine a rank pulls an output row its owner has not written yet.
    assert _violates(*ep_model(2, 2, barrier_before_combine=False), 2)


# ---- GEMM -> reduce-scatter without a barrier (csrc/fused/tp_fused.cu) -------------------------------------------------
# One tile per owner. In call k (parity p) a rank stores its partial of every tile into the owner's staging
# [p][source], remote owners first, and bumps the owner's counter [p]; then it waits until its own counter [p] shows
# all n partials of this call and sums them. Counters only grow: the target of call k is n * (calls of that parity so
# far). Nothing else orders the ranks; the claim is that two staging halves are enough.
def gemm_rs_model(n, ncalls, nbufs=2):
    def step(st, pid):
        procs, stage, cnt = st
        k, pc, idx = procs[pid]
        if k > ncalls:
            return None
        p = k % nbufs
        target = n * ((k + nbufs - 1) // nbufs) if nbufs == 2 else n * k

        def upd(t, i, v):
            return t[:i] + (v,) + t[i + 1:]

        if pc == 0:  # store the partial of the tile owned by rank (pid + 1 + idx) % n
            owner = (pid + 1 + idx) % n
            return (upd(procs, pid, (k, 1, idx)), upd(stage, (owner * nbufs + p) * n + pid, (pid, k)), cnt)
        if pc == 1:  # red.release.sys.add on the owner's counter
            owner = (pid + 1 + idx) % n
            cell = owner * nbufs + p
            nxt = (k, 0, idx + 1) if idx + 1 < n else (k, 2, 0)
            return (upd(procs, pid, nxt), stage, upd(cnt, cell, cnt[cell] + 1))
        if pc == 2:  # reducer: wait for the counter, then read the n partials one by one
            if cnt[pid * nbufs + p] < target:
                return None
            return (upd(procs, pid, (k, 3, 0)), stage, cnt)
        got = stage[(pid * nbufs + p) * n + idx]
        assert got == (idx, k), f"rank {pid} call {k}: partial of rank {idx} is {got}"
        nxt = (k, 3, idx + 1) if idx + 1 < n else (k + 1, 0, 0)
        return (upd(procs, pid, nxt), stage, cnt)

    initial = (tuple((1, 0, 0) for _ in range(n)), tuple((None, 0) for _ in range(n * nbufs * n)), tuple(0 for _ in range(n * nbufs)))
    return initial, step, (lambda st: all(pr[0] > ncalls for pr in st[0]))


def test_gemm_reduce_scatter_needs_no_barrier_with_two_staging_halves():
    for n, ncalls in [(2, 6), (3, 3)]:
        initial, step, done = gemm_rs_model(n, ncalls)
        states, deadlocks = explore(initial, step, done, n)
        assert deadlocks == 0 and states > 20 * ncalls


def test_gemm_rs_checker_finds_the_single_half_overwrite():
    assert _violates(*gemm_rs_model(2, 3, nbufs=1), 2)


# ---- all-gather -> GEMM (tp_fused.cu, tp_fused_fp8.cu): pulled row blocks behind sequence-numbered flags -------------
# Per rank two actors of one kernel launch: the communication CTA (barrier: every shard is in place; pull each peer's
# block into the local copy; publish the block's flag with the call's sequence number; barrier: the peers are done
# reading my shard) and a GEMM CTA (own block at once, a peer's block after its flag reached the sequence number).
# Launches of one rank are stream-ordered: call k + 1 starts, and the application overwrites the rank's own shard with
# the next activations, only after both actors of call k are done. A block's content is modelled as the number of the
# call it belongs to; a GEMM CTA must only ever multiply blocks of its own call.
def ag_gemm_model(n, ncalls, end_barrier=True):
    def upd(t, i, v):
        return t[:i] + (v,) + t[i + 1:]

    def step(st, pid):
        comm, gemm, shard, local, flag, bar_a, bar_b = st
        r = pid % n
        if pid < n:  # communication CTA of rank r
            k, pc, idx = comm[r]
            if k > ncalls:
                return None
            if pc == 0:  # launch: previous kernel of this rank complete; the application has written the shard of call k
                if gemm[r][0] < k:  # the GEMM CTA of call k - 1 is still running
                    return None
                return (upd(comm, r, (k, 1, 0)), gemm, upd(shard, r, k), local, flag, upd(bar_a, r, k), bar_b)
            if pc == 1:  # first barrier
                if any(b < k for b in bar_a):
                    return None
                return (upd(comm, r, (k, 2, 0)), gemm, shard, local, flag, bar_a, bar_b)
            if pc == 2:  # pull the block of peer (r + 1 + idx) % n: read the owner's shard as it is now
                peer = (r + 1 + idx) % n
                return (upd(comm, r, (k, 3, idx)), gemm, shard, upd(local, r * n + peer, shard[peer]), flag, bar_a, bar_b)
            if pc == 3:  # publish its flag
                peer = (r + 1 + idx) % n
                nxt = (k, 2, idx + 1) if idx + 2 < n else (k, 4, 0)
                return (upd(comm, r, nxt), gemm, shard, local, upd(flag, r * n + peer, k), bar_a, bar_b)
            if pc == 4:  # second barrier: arrive
                return (upd(comm, r, (k, 5, 0)), gemm, shard, local, flag, bar_a, upd(bar_b, r, k))
            if end_barrier and any(b < k for b in bar_b):
                return None
            return (upd(comm, r, (k + 1, 0, 0)), gemm, shard, local, flag, bar_a, bar_b)
        k, idx = gemm[r]
        if k > ncalls or comm[r][0] < k or (comm[r][0] == k and comm[r][1] == 0):
            return None  # finished, or the kernel of call k has not been launched on this rank
        owner = (r + idx) % n
        if owner == r:
            got = shard[r]
        else:
            if flag[r * n + owner] < k:
                return None
            got = local[r * n + owner]
        assert got == k, f"rank {r} call {k}: block of rank {owner} belongs to call {got}"
        nxt = (k, idx + 1) if idx + 1 < n else (k + 1, 0)
        return (comm, upd(gemm, r, nxt), shard, local, flag, bar_a, bar_b)

    zeros = tuple(0 for _ in range(n))
    initial = (tuple((1, 0, 0) for _ in range(n)), tuple((1, 0) for _ in range(n)), zeros, tuple(0 for _ in range(n * n)),
               tuple(0 for _ in range(n * n)), zeros, zeros)
    return initial, step, (lambda st: all(c[0] > ncalls for c in st[0]) and all(g[0] > ncalls for g in st[1]))


def test_all_gather_gemm_reads_only_blocks_of_its_own_call():
    for n, ncalls in [(2, 4), (3, 2)]:
        initial, step, done = ag_gemm_model(n, ncalls)
        states, deadlocks = explore(initial, step, done, 2 * n)
        assert deadlocks == 0 and states > 30 * ncalls


def test_all_gather_gemm_checker_finds_the_missing_closing_barrier():
    """Without the second barrier a fast rank starts its next call and overwrites its shard while a peer still pulls it."""
    assert _violates(*ag_gemm_model(2, 2, end_barrier=False), 4)


# ---- shared-memory ring of bulk asynchronous peer loads (kStagedReduce, peer-load path) ------------------------------
# A group of threads walks tiles 0..K-1 through S stages. Thread 0 issues tile i into stage i % S (arming the stage's
# mbarrier; the copy engine completes it at any later time, which stores the data and flips the barrier's phase);
# every thread waits for tile i on parity (i / S) & 1, thread 0 then issues tile i + S - 1, all reduce the tile, and all
# meet at a named barrier. Before the loop thread 0 has issued tiles 0..S-2.
def bulk_ring_model(nthreads, stages, tiles, issue_after_wait=True, lookahead=None):
    ahead = stages - 1 if lookahead is None else lookahead

    def step(st, pid):
        threads, armed, phase, data, arrived, gen = st
        # the last "process" is the copy engine: it completes any armed stage
        if pid >= nthreads:
            s = pid - nthreads
            if armed[s] is None:
                return None
            return (threads, armed[:s] + (None,) + armed[s + 1:], phase[:s] + (phase[s] + 1,) + phase[s + 1:], data[:s] + (armed[s],) + data[s + 1:], arrived, gen)
        i, pc, mygen = threads[pid]
        if i >= tiles:
            return None

        def upd(t, k, v):
            return t[:k] + (v,) + t[k + 1:]

        def issue(armed_, phase_, tile):
            s = tile % stages
            assert armed_[s] is None, f"tile {tile}: stage {s} armed while tile {armed_[s]} is still in flight"
            return upd(armed_, s, tile)

        s = i % stages
        if pc == 0:  # mbarrier.try_wait.parity: passes when the current phase's parity differs from the awaited one
            if (phase[s] & 1) == ((i // stages) & 1):
                return None
            return (upd(threads, pid, (i, 1, mygen)), armed, phase, data, arrived, gen)
        if pc == 1:  # thread 0 refills the stage everybody left at the end of the previous iteration
            armed2 = armed
            if pid == 0 and issue_after_wait and i + ahead < tiles:
                armed2 = issue(armed, phase, i + ahead)
            return (upd(threads, pid, (i, 2, mygen)), armed2, phase, data, arrived, gen)
        if pc == 2:  # reduce the tile out of shared memory
            assert data[s] == i, f"thread {pid} tile {i}: stage {s} holds tile {data[s]}"
            return (upd(threads, pid, (i, 3, mygen)), armed, phase, data, arrived, gen)
        if pc == 3:  # arrive at the named barrier
            arrived2 = arrived + 1
            if arrived2 == nthreads:
                return (upd(threads, pid, (i, 4, mygen)), armed, phase, data, 0, gen + 1)
            return (upd(threads, pid, (i, 4, mygen)), armed, phase, data, arrived2, gen)
        if gen == mygen:  # pc == 4: leave the barrier once its generation has advanced
            return None
        return (upd(threads, pid, (i + 1, 0, gen)), armed, phase, data, arrived, gen)

    armed = [None] * stages
    for tile in range(min(ahead, tiles)):
        armed[tile % stages] = tile
    initial = (tuple((0, 0, 0) for _ in range(nthreads)), tuple(armed), tuple(0 for _ in range(stages)), tuple(-1 for _ in range(stages)), 0, 0)
    return initial, step, (lambda st: all(t[0] >= tiles for t in st[0]))


def test_bulk_load_ring_never_overwrites_or_misreads_a_stage():
    for nthreads, stages, tiles in [(2, 4, 11), (3, 4, 9), (2, 2, 6)]:
        initial, step, done = bulk_ring_model(nthreads, stages, tiles)
        states, deadlocks = explore(initial, step, done, nthreads + stages)
        assert deadlocks == 0 and states > 50


def test_bulk_ring_checker_finds_a_refill_that_is_one_stage_too_eager():
    # Keeping S tiles in flight instead of S - 1 refills the stage the other threads may still be reading.
    assert _violates(*bulk_ring_model(2, 4, 9, lookahead=4), 2 + 4)


# ---- the block-scaled fp8 GEMM's pipeline (csrc/fused/gemm_fp8_sm100.cu) ---------------------------------------------
# Producer thread, MMA thread and W epilogue warps over N K-blocks, S shared-memory stages and two accumulators:
#   producer j: wait empty[s] (parity ph ^ 1) ; arm full[s] and start the TMA loads (complete later) ; s, ph advance
#   MMA      j: wait partEmpty[b] (parity bph ^ 1) ; wait full[s] (parity ph) ; issue the MMAs of block j into accumulator b ;
#               commit -> empty[s] and partFull[b] arrive when the MMAs have finished (later)
#   epilogue j: wait partFull[b] (parity bph) ; read accumulator b ; arrive on partEmpty[b] (W arrivals complete a phase)
# with b = j & 1, bph = (j >> 1) & 1, s = j % S, ph = (j / S) & 1. A barrier is its count of completed phases; a parity wait
# passes when the current phase's parity differs from the awaited one.
def fp8_pipeline_model(nblocks, stages, warps, wait_part_empty=True):
    P, M = 0, 1

    def step(st, pid):
        pj, mj, mpc, ej, epc, full, empty, pfull, pempty, pe_arrivals, smem, tma, tmem, mma, readers = st

        def upd(t, k, v):
            return t[:k] + (v,) + t[k + 1:]

        if pid == P:
            if pj >= nblocks:
                return None
            s, ph = pj % stages, (pj // stages) & 1
            if (empty[s] & 1) == (ph ^ 1):
                return None
            assert tma[s] is None and mma[s] is None, f"producer block {pj}: stage {s} is still in use"
            return (pj + 1, mj, mpc, ej, epc, full, empty, pfull, pempty, pe_arrivals, smem, upd(tma, s, pj), tmem, mma, readers)
        if pid == M:
            if mj >= nblocks:
                return None
            s, ph, b, bph = mj % stages, (mj // stages) & 1, mj & 1, (mj >> 1) & 1
            if mpc == 0:
                if wait_part_empty and (pempty[b] & 1) == (bph ^ 1):
                    return None
                return (pj, mj, 1, ej, epc, full, empty, pfull, pempty, pe_arrivals, smem, tma, tmem, mma, readers)
            if (full[s] & 1) == ph:
                return None
            assert smem[s] == mj, f"MMA block {mj}: stage {s} holds block {smem[s]}"
            assert mj < 2 or readers[b] == warps, f"MMA block {mj}: accumulator {b} overwritten while {warps - readers[b]} warp(s) still read block {mj - 2}"
            return (pj, mj + 1, 0, ej, epc, full, empty, pfull, pempty, pe_arrivals, smem, tma, tmem, upd(mma, s, mj), upd(readers, b, 0))
        if pid < 2 + warps:  # epilogue warp w
            w = pid - 2
            j = ej[w]
            if j >= nblocks:
                return None
            b, bph = j & 1, (j >> 1) & 1
            if epc[w] == 0:
                if (pfull[b] & 1) == bph:
                    return None
                return (pj, mj, mpc, ej, upd(epc, w, 1), full, empty, pfull, pempty, pe_arrivals, smem, tma, tmem, mma, readers)
            assert tmem[b] == j, f"warp {w} block {j}: accumulator {b} holds block {tmem[b]}"
            arr = pe_arrivals[b] + 1
            pempty2, arr2 = (upd(pempty, b, pempty[b] + 1), 0) if arr == warps else (pempty, arr)
            return (pj, mj, mpc, upd(ej, w, j + 1), upd(epc, w, 0), full, empty, pfull, pempty2, upd(pe_arrivals, b, arr2), smem, tma, tmem, mma,
                    upd(readers, b, readers[b] + 1))
        k = pid - 2 - warps
        if k < stages:  # the TMA unit finishes the loads of a stage
            if tma[k] is None:
                return None
            return (pj, mj, mpc, ej, epc, upd(full, k, full[k] + 1), empty, pfull, pempty, pe_arrivals, upd(smem, k, tma[k]), upd(tma, k, None), tmem, mma, readers)
        s = k - stages  # the tensor core finishes the MMAs that read stage s: both commits arrive
        if mma[s] is None:
            return None
        j = mma[s]
        b = j & 1
        return (pj, mj, mpc, ej, epc, full, upd(empty, s, empty[s] + 1), upd(pfull, b, pfull[b] + 1), pempty, pe_arrivals, smem, tma, upd(tmem, b, j),
                upd(mma, s, None), readers)

    z = tuple
    initial = (0, 0, 0, z(0 for _ in range(warps)), z(0 for _ in range(warps)), z(0 for _ in range(stages)), z(0 for _ in range(stages)), (0, 0), (0, 0), (0, 0),
               z(-1 for _ in range(stages)), z(None for _ in range(stages)), (-1, -1), z(None for _ in range(stages)), (0, 0))
    return initial, step, (lambda st: st[0] >= nblocks and st[1] >= nblocks and all(e >= nblocks for e in st[3]))


def test_fp8_gemm_pipeline_has_no_deadlock_and_no_accumulator_or_stage_hazard():
    for nblocks, stages, warps in [(7, 3, 2), (6, 2, 2), (5, 3, 3)]:
        initial, step, done = fp8_pipeline_model(nblocks, stages, warps)
        states, deadlocks = explore(initial, step, done, 2 + warps + 2 * stages)
        assert deadlocks == 0 and states > 100


def test_fp8_pipeline_checker_finds_the_missing_accumulator_wait():
    # Without the wait on partEmpty the third block is multiplied into an accumulator the epilogue still reads.
    assert _violates(*fp8_pipeline_model(5, 3, 2, wait_part_empty=False), 2 + 2 + 6)
