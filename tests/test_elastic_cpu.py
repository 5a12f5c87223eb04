"""Failure detection and elastic recovery on CPU ranks: a rank leaves (or dies silently) between
steps, the survivors learn of it through the store, re-form the group without it, re-shard the
last checkpoint to the smaller world and finish with exactly the parameters an undisturbed run has."""
import multiprocessing as mp
import os
import socket
import sys
import time
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

NUMEL, SAMPLES, STEPS, LEAVE_AFTER = 37, 6, 5, 2
LR, B1, B2, EPS, WD = 0.05, 0.9, 0.95, 1e-8, 0.1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _problem():
    import torch

    g = torch.Generator().manual_seed(5)
    A = torch.randn(SAMPLES, 11, NUMEL, generator=g, dtype=torch.float64)
    b = torch.randn(SAMPLES, 11, generator=g, dtype=torch.float64)
    p0 = torch.randn(NUMEL, generator=g, dtype=torch.float64)
    return A, b, p0


def _grad(A, b, p, idx):
    import torch

    gs = [A[i].t() @ (A[i] @ p - b[i]) for i in idx]
    return torch.stack(gs).mean(0)


def _adamw(p, m, v, g, step):
    m.mul_(B1).add_(g, alpha=1 - B1)
    v.mul_(B2).addcmul_(g, g, value=1 - B2)
    upd = (m / (1 - B1 ** step)) / ((v / (1 - B2 ** step)).sqrt() + EPS)
    p.sub_(LR * (upd + WD * p))


def _reference():
    import torch

    A, b, p0 = _problem()
    p, m, v = p0.clone(), torch.zeros(NUMEL, dtype=torch.float64), torch.zeros(NUMEL, dtype=torch.float64)
    for step in range(1, STEPS + 1):
        _adamw(p, m, v, _grad(A, b, p, range(SAMPLES)), step)
    return p


def _worker(orig_rank, world0, port, ckpt, mode, q):
    import traceback

    try:
        import torch
        import torch.distributed as dist

        from rocm_systems_b200.utils import checkpoint, elastic

        store = dist.TCPStore("127.0.0.1", port, world0, is_master=(orig_rank == 0), wait_for_workers=False)
        dist.init_process_group("gloo", store=dist.PrefixStore("gen0", store), rank=orig_rank, world_size=world0)
        hb = elastic.Heartbeat(store, orig_rank, world0, interval=0.1, timeout=1.0).start()
        A, b, p0 = _problem()
        rank, world = orig_rank, world0

        def layout(w):
            return (NUMEL + w - 1) // w

        sn = layout(world)
        full0 = torch.zeros(sn * world, dtype=torch.float64)
        full0[:NUMEL] = p0
        shard = {"master": full0[rank * sn:(rank + 1) * sn].clone(), "m": torch.zeros(sn, dtype=torch.float64), "v": torch.zeros(sn, dtype=torch.float64)}
        step, generation = 0, 0
        while step < STEPS:
            # ---- step boundary: who is still there? ----
            if hb.lost():
                generation += 1
                rank, world = elastic.reform_group(store, hb, generation, backend="gloo")
                assert world == world0 - 1 and rank >= 0
                sn = layout(world)
                sd = checkpoint.load_for(ckpt, rank, world, {"p": sn})
                shard, step = sd["units"]["p"], sd["step"]
            parts = [torch.empty(sn, dtype=torch.float64) for _ in range(world)]
            dist.all_gather(parts, shard["master"])
            p = torch.cat(parts)[:NUMEL]
            g = _grad(A, b, p, range(rank, SAMPLES, world))
            dist.all_reduce(g)
            g /= world
            gp = torch.zeros(sn * world, dtype=torch.float64)
            gp[:NUMEL] = g
            step += 1
            _adamw(shard["master"], shard["m"], shard["v"], gp[rank * sn:(rank + 1) * sn], step)
            checkpoint.save_sharded({"step": step, "world": world, "rank": rank, "units": {"p": shard}}, ckpt, {"p": NUMEL})
            dist.barrier()  # the checkpoint of this step is complete on every rank
            if orig_rank == world0 - 1 and step == LEAVE_AFTER and generation == 0:
                if mode == "leave":
                    hb.leave()
                    dist.destroy_process_group()
                    q.put((orig_rank, None, "left"))
                    return
                q.put((orig_rank, None, "died"))
                q.close()
                q.join_thread()
                os._exit(0)  # no goodbye: the others must notice the silence
            if step == LEAVE_AFTER and generation == 0:
                t0 = time.monotonic()  # give the detector time to see the loss before the next collective
                while not hb.lost() and time.monotonic() - t0 < 10:
                    time.sleep(0.05)
        parts = [torch.empty(sn, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(parts, shard["master"])
        final = torch.cat(parts)[:NUMEL]
        hb.stop()
        dist.destroy_process_group()
        q.put((orig_rank, None, final.tolist()))
    except Exception:  # noqa: BLE001
        q.put((orig_rank, traceback.format_exc(), None))


@pytest.mark.parametrize("mode", ["leave", "die"])
def test_rank_lost_between_steps_job_continues(tmp_path, mode):
    import torch

    ctx = mp.get_context("spawn")
    port, world = _free_port(), 3
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, str(tmp_path / "ckpt"), mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    errs = [r for r in res if r[1]]
    assert not errs, errs
    finals = [torch.tensor(r[2], dtype=torch.float64) for r in res if isinstance(r[2], list)]
    assert len(finals) == 2
    want = _reference()
    for f in finals:
        assert torch.allclose(f, want, rtol=1e-12, atol=1e-12), (f - want).abs().max()


def test_reshard_roundtrip_and_padding():
    import torch

    from rocm_systems_b200.utils import checkpoint

    flat = torch.arange(10, dtype=torch.float32)
    old = [torch.cat([flat, torch.zeros(2)])[i * 4:(i + 1) * 4] for i in range(3)]   # world 3, shard 4, 2 pad
    new = [checkpoint.reshard_unit(old, 10, r, 5) for r in range(2)]
    assert torch.equal(torch.cat(new), flat)
    wide = [checkpoint.reshard_unit(old, 10, r, 3) for r in range(4)]                    # world 4, shard 3, 2 pad
    assert torch.equal(torch.cat(wide)[:10], flat) and torch.equal(torch.cat(wide)[10:], torch.zeros(2))


def test_incomplete_checkpoint_is_refused(tmp_path):
    import torch

    from rocm_systems_b200.utils import checkpoint

    sd = {"step": 3, "world": 2, "rank": 0, "units": {"p": {k: torch.zeros(4) for k in checkpoint.KEYS}}}
    with pytest.raises(checkpoint.CheckpointNotCommitted):              # rank 1 never writes: rank 0 gives up, nothing is committed
        checkpoint.save_sharded(sd, str(tmp_path), {"p": 7}, commit_timeout_s=0.2)
    assert checkpoint.complete_steps(str(tmp_path)) == []
    with pytest.raises(FileNotFoundError):
        checkpoint.load_shards(str(tmp_path))


def test_rank_dying_mid_save_leaves_the_previous_step_loadable(tmp_path):
    """Step 3 is saved by both ranks and committed. During the save of step 5 rank 1 dies after rank 0 wrote its shard
    and before the commit marker exists: loading still gives step 3 on every rank, a shard of the wrong step is refused,
    and the next complete save cleans the half-written step up."""
    import json

    import torch

    from rocm_systems_b200.utils import checkpoint

    d = str(tmp_path)

    def state(step, rank, fill):
        return {"step": step, "world": 2, "rank": rank, "units": {"p": {k: torch.full((4,), float(fill)) for k in checkpoint.KEYS}}}

    checkpoint.save_sharded(state(3, 1, 31), d, {"p": 7})             # rank 1 first: it returns at once, rank 0 commits
    checkpoint.save_sharded(state(3, 0, 30), d, {"p": 7})
    assert checkpoint.complete_steps(d) == [3]
    with pytest.raises(checkpoint.CheckpointNotCommitted):
        checkpoint.save_sharded(state(5, 0, 50), d, {"p": 7}, commit_timeout_s=0.2)   # rank 1 is gone
    assert checkpoint.all_steps(d) == [3, 5] and checkpoint.complete_steps(d) == [3]
    for r in range(2):                                                  # both ranks resume from the same, complete step
        sd = checkpoint.load_for(d, r, 2, {"p": 4})
        assert sd["step"] == 3 and sd["rank"] == r and float(sd["units"]["p"]["master"][0]) == 30 + r
    one = checkpoint.load_for(d, 0, 1, {"p": 8})                        # and a smaller world re-shards that step
    assert one["step"] == 3 and one["units"]["p"]["m"].tolist() == [30.0] * 4 + [31.0] * 3 + [0.0]
    # a shard that claims another step than the commit marker is refused on the same-world path too
    torch.save(state(4, 1, 41), tmp_path / "step-3" / "rank1.pt")
    with pytest.raises(ValueError):
        checkpoint.load_for(d, 1, 2, {"p": 4})
    torch.save(state(3, 1, 31), tmp_path / "step-3" / "rank1.pt")
    # the next complete save commits, keeps the newest `keep` steps and removes the half-written one
    checkpoint.save_sharded(state(7, 1, 71), d, {"p": 7})
    checkpoint.save_sharded(state(7, 0, 70), d, {"p": 7}, keep=1)
    assert checkpoint.all_steps(d) == [7] and json.loads((tmp_path / "step-7" / "meta.json").read_text())["step"] == 7
    # files are read with weights_only=True: a pickled object is refused instead of executed
    torch.save({"step": 7, "world": 2, "rank": 1, "units": {"p": {"master": object()}}}, tmp_path / "step-7" / "rank1.pt")
    with pytest.raises(Exception):
        checkpoint.load_for(d, 1, 2, {"p": 4})
