"""A 4-layer MLP trained as a pipeline: one stage per rank, 1F1B schedule, SGD.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/pipeline_1f1b.py
    ... --nproc-per-node 4 examples/pipeline_1f1b.py --device cuda      # one GPU per stage, b200coll backend

Every rank builds the whole model from one seed and keeps its own slice of layers, so the result can be
compared with the unsplit model: the last rank prints both losses after every step.
"""
import argparse
import copy
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from rocm_systems_b200.parallel.pp import PipelineStage  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", choices=["cpu", "cuda"], default="cpu")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--micro", type=int, default=8)
    ap.add_argument("--width", type=int, default=64)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if a.device == "cuda":
        from rocm_systems_b200.parallel import init_process_group

        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        init_process_group()
        dev = torch.device("cuda", torch.cuda.current_device())
    else:
        dist.init_process_group("gloo")
        dev = torch.device("cpu")

    torch.manual_seed(0)
    layers_per_stage = 2
    full = [torch.nn.Sequential(torch.nn.Linear(a.width, a.width), torch.nn.Tanh()) for _ in range(world * layers_per_stage)]
    mine = torch.nn.Sequential(*full[rank * layers_per_stage:(rank + 1) * layers_per_stage]).to(dev)
    reference = copy.deepcopy(torch.nn.Sequential(*full)).to(dev)
    opt = torch.optim.SGD(mine.parameters(), lr=0.1)
    ref_opt = torch.optim.SGD(reference.parameters(), lr=0.1)
    stage = PipelineStage(mine, rank, world, act_shape=(4, a.width), device=dev)
    loss_fn = torch.nn.functional.mse_loss
    worst = 0.0
    for step in range(a.steps):
        g = torch.Generator().manual_seed(100 + step)
        xs = [torch.randn(4, a.width, generator=g) for _ in range(a.micro)]
        ys = [torch.randn(4, a.width, generator=g) for _ in range(a.micro)]
        opt.zero_grad()
        losses = stage.run(xs, ys, loss_fn, n_micro=a.micro, schedule="1f1b")
        opt.step()
        # the same step on the unsplit model
        ref_opt.zero_grad()
        ref_losses = []
        for x, y in zip(xs, ys):
            loss = loss_fn(reference(x.to(dev)), y.to(dev)) / a.micro
            loss.backward()
            ref_losses.append(float(loss.detach()) * a.micro)
        ref_opt.step()
        if stage.last:
            diff = max(abs(p - q) for p, q in zip(losses, ref_losses))
            worst = max(worst, diff)
            print(f"step {step}: pipeline loss {sum(losses) / len(losses):.6f}  unsplit {sum(ref_losses) / len(ref_losses):.6f}  "
                  f"max |diff| {diff:.2e}  activations alive at once on this stage: {stage.peak_alive}", flush=True)
    ok = worst < 1e-4
    if stage.last:
        print("pipeline_1f1b OK" if ok else "pipeline_1f1b MISMATCH", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
