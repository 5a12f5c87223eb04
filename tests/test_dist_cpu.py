"""Plumbing correctness on CPU: world_size 2, fp32 tensors of 1,048,576 elements, values
uniform[-1, 1] from seed = rank, through the process group this package sets up (CUDA tensors go
to b200coll, CPU tensors to gloo). Results are checked against a numpy reduction of both ranks'
inputs at rtol 1e-6.
"""
import multiprocessing as mp
import os
import socket

import numpy as np
import pytest

N = 1 << 20


def _inputs(rank):
    rng = np.random.default_rng(rank)
    return rng.uniform(-1.0, 1.0, N).astype(np.float32)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world)})
    import torch
    import torch.distributed as dist

    from rocm_systems_b200.parallel import init_process_group

    try:
        init_process_group()
        xs = [_inputs(r) for r in range(world)]
        mine = torch.from_numpy(xs[rank].copy())
        errs = []

        def close(name, got, want):
            if not np.allclose(got.numpy(), want, rtol=1e-6, atol=1e-6):
                errs.append(name)

        t = mine.clone()
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        close("all_reduce_sum", t, xs[0] + xs[1])
        t = mine.clone()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        close("all_reduce_max", t, np.maximum(xs[0], xs[1]))
        out = torch.empty(N // world)
        dist.reduce_scatter_tensor(out, mine.clone(), op=dist.ReduceOp.SUM)
        close("reduce_scatter", out, (xs[0] + xs[1])[rank * (N // world):(rank + 1) * (N // world)])
        gathered = torch.empty(N * world)
        dist.all_gather_into_tensor(gathered, mine)
        close("all_gather", gathered, np.concatenate(xs))
        b = mine.clone() if rank == 0 else torch.zeros(N)
        dist.broadcast(b, src=0)
        close("broadcast", b, xs[0])
        a2a = torch.empty(N)
        dist.all_to_all_single(a2a, mine)
        half = N // world
        close("all_to_all", a2a, np.concatenate([xs[s][rank * half:(rank + 1) * half] for s in range(world)]))
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, errs))
    except Exception as e:  # noqa: BLE001
        q.put((rank, [f"exception: {type(e).__name__}: {e}"]))


def test_cpu_gloo_world2_sweep():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=180) for _ in range(2))
    for p in ps:
        p.join(timeout=30)
    assert res[0] == [] and res[1] == [], res
