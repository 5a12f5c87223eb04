"""One rank of the torch.distributed (backend b200coll) check on CUDA tensors."""
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from rocm_systems_b200.parallel import init_process_group  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    init_process_group(device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    fails = []

    def expect(name, got, want):
        if not torch.equal(got, want.to(got.dtype)):
            fails.append(name)

    n = 1 << 18
    base = [torch.arange(n, device=dev, dtype=torch.float32) % 7 + r for r in range(world)]
    t = base[rank].clone()
    dist.all_reduce(t)
    expect("all_reduce", t, sum(base))
    t = base[rank].clone().to(torch.bfloat16)
    w = dist.all_reduce(t, op=dist.ReduceOp.MAX, async_op=True)
    w.wait()
    expect("all_reduce_max_bf16_async", t, torch.stack(base).max(0).values)
    t = base[rank].clone()
    dist.all_reduce(t, op=dist.ReduceOp.AVG)
    expect("all_reduce_avg", t, sum(base) / world)
    out = torch.empty(n // world, device=dev)
    dist.reduce_scatter_tensor(out, base[rank].clone())
    expect("reduce_scatter_tensor", out, sum(base)[rank * (n // world):(rank + 1) * (n // world)])
    g = torch.empty(n * world, device=dev)
    dist.all_gather_into_tensor(g, base[rank])
    expect("all_gather_into_tensor", g, torch.cat(base))
    lst = [torch.empty(n, device=dev) for _ in range(world)]
    dist.all_gather(lst, base[rank])
    expect("all_gather_list", torch.cat(lst), torch.cat(base))
    outs = torch.empty(n // world, device=dev)
    dist.reduce_scatter(outs, list(base[rank].clone().chunk(world)))
    expect("reduce_scatter_list", outs, sum(base)[rank * (n // world):(rank + 1) * (n // world)])
    b = base[0].clone() if rank == 0 else torch.zeros(n, device=dev)
    dist.broadcast(b, src=0)
    expect("broadcast", b, base[0])
    r = base[rank].clone()
    dist.reduce(r, dst=world - 1)
    if rank == world - 1:
        expect("reduce", r, sum(base))
    a2a = torch.empty(n, device=dev)
    dist.all_to_all_single(a2a, base[rank])
    per = n // world
    expect("all_to_all_single", a2a, torch.cat([base[s][rank * per:(rank + 1) * per] for s in range(world)]))
    # uneven splits: rank s sends (d + 1) * k rows to rank d
    k = 10
    in_split = [(d + 1) * k for d in range(world)]
    out_split = [(rank + 1) * k for _ in range(world)]
    src = [torch.arange(sum(in_split) * 4, device=dev, dtype=torch.float32).view(-1, 4) + 1000 * s for s in range(world)]
    o = torch.empty(sum(out_split), 4, device=dev)
    dist.all_to_all_single(o, src[rank], out_split, in_split)
    want = torch.cat([src[s][sum(in_split[:rank]):sum(in_split[:rank]) + in_split[rank]] for s in range(world)])
    expect("all_to_all_single_uneven", o, want)
    if world >= 2:
        if rank == 0:
            dist.send(base[0], dst=1)
        elif rank == 1:
            rr = torch.empty(n, device=dev)
            dist.recv(rr, src=0)
            expect("send_recv", rr, base[0])
        ops = [dist.P2POp(dist.isend, base[rank], (rank + 1) % world)]
        rb = torch.empty(n, device=dev)
        ops.append(dist.P2POp(dist.irecv, rb, (rank - 1) % world))
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        expect("batch_isend_irecv", rb, base[(rank - 1) % world])
    dist.barrier()

    # A small data-parallel model: DDP gradients must match the averaged local gradients.
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 8)).to(dev)
    ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local])
    xs = [torch.randn(16, 64, generator=torch.Generator().manual_seed(100 + r)).to(dev) for r in range(world)]
    ddp(xs[rank]).square().mean().backward()
    got = [p.grad.clone() for p in model.parameters()]
    ref = [torch.zeros_like(p) for p in model.parameters()]
    for r in range(world):
        model.zero_grad()
        model(xs[r]).square().mean().backward()
        for a, p in zip(ref, model.parameters()):
            a += p.grad / world
    for i, (a, b2) in enumerate(zip(got, ref)):
        if not torch.allclose(a, b2, rtol=1e-4, atol=1e-6):
            fails.append(f"ddp_grad_{i}")
    torch.cuda.synchronize()
    flag = torch.tensor([len(fails)], device=dev, dtype=torch.int32)
    dist.all_reduce(flag)
    if fails:
        print(f"[rank {rank}] dist_worker FAILURES: {fails}", flush=True)
    elif rank == 0:
        print(f"dist_worker OK on {world} ranks", flush=True)
    dist.destroy_process_group()
    sys.exit(1 if int(flag.item()) else 0)


if __name__ == "__main__":
    main()
