"""Train a small Llama with the FSDP engine on every GPU of the box, checkpoint, and resume.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_llama_fsdp.py --steps 20
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rocm_systems_b200.comm import init_from_env  # noqa: E402
from rocm_systems_b200.models.llama import LlamaConfig, LlamaTrainer  # noqa: E402
from rocm_systems_b200.utils import checkpoint, hang_dump, markers, schedule  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--ckpt", default="ckpt_example")
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--model", default="", help="a name LlamaConfig.by_name knows (llama3-8b, llama3.2-1b, ...); default: a 150M-parameter model")
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    comm = init_from_env(device=local) if world > 1 else None
    cfg = LlamaConfig.by_name(a.model) if a.model else LlamaConfig(vocab=8192, hidden=1024, layers=8, heads=16, kv_heads=4, ffn=4096, seq_len=1024)
    if comm is None or comm.rank == 0:
        est = cfg.memory_per_gpu_gib(world, 2 * cfg.seq_len)
        print(f"{cfg.param_count() / 1e9:.2f} B parameters; estimated {est['total']:.1f} GiB per GPU ({est['state']:.1f} state, {est['activations']:.1f} activations)", flush=True)
    trainer = LlamaTrainer(cfg, comm, torch.device("cuda", local))
    lr_at = schedule.warmup_cosine(peak=a.lr, warmup=a.warmup, total=max(a.steps, a.warmup + 1), floor=a.lr / 10)
    if a.resume:
        checkpoint.load_engine(trainer.engine, a.ckpt)  # re-shards when the world size changed
    g = torch.Generator().manual_seed(1 + (comm.rank if comm else 0))
    hang_dump.arm(600, comms=[comm] if comm else [])  # ten minutes without a finished step: say where everything is
    for step in range(a.steps):
        tok = torch.randint(0, cfg.vocab, (2, cfg.seq_len), generator=g).pin_memory()
        trainer.engine.opt.lr = lr_at(trainer.engine.step_count)  # the engine reads the rate at every unit's update
        with markers.range(f"step {step}"):  # shows up in traces taken with tools.prof --marker-trace
            loss = trainer.step(tok, tok.roll(-1, 1).pin_memory())
        hang_dump.kick()
        if (comm is None or comm.rank == 0) and step % 5 == 0:
            print(f"step {step}: loss {loss:.4f}", flush=True)
    hang_dump.disarm()
    checkpoint.save_engine(trainer.engine, a.ckpt)
    if comm is not None:
        comm.host_barrier()
        comm.destroy()


if __name__ == "__main__":
    main()
