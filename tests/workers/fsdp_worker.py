"""One rank of the FSDP check: a tiny Llama trained on N ranks (one batch per rank) must follow
the same loss curve as one rank training on all the batches together."""
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402

from rocm_systems_b200.comm import init_from_env  # noqa: E402
from rocm_systems_b200.models.llama import LlamaConfig, LlamaTrainer  # noqa: E402
from rocm_systems_b200.parallel.fsdp import AdamWConfig  # noqa: E402


def main():
    comm = init_from_env()
    rank, world = comm.rank, comm.nranks
    dev = comm.device
    cfg = LlamaConfig.tiny(64)
    fused = os.environ.get("FSDP_FUSED_RS", "1") == "1"
    sym = os.environ.get("FSDP_SYM_SHARDS", "1") == "1"   # shards and gradient buffers in symmetric memory (zero-copy collectives)
    ce = {"1": True, "0": False}.get(os.environ.get("FSDP_COPY_ENGINE_GATHER", ""), None)   # parameter all-gather by copy engines (1), by the kernel (0), or the default
    clip = float(os.environ.get("FSDP_CLIP", "0"))         # > 0: global-norm clipping to this value on both trainers
    opt = (lambda: AdamWConfig(max_grad_norm=clip)) if clip > 0 else (lambda: None)
    sharded = LlamaTrainer(cfg, comm, dev, opt=opt(), seed=3, fused_rs=fused, sym_shards=sym, copy_engine_gather=ce)
    single = LlamaTrainer(cfg, None, dev, opt=opt(), seed=3)
    g = torch.Generator().manual_seed(5)
    steps = 6
    toks = [torch.randint(0, cfg.vocab, (world, cfg.seq_len), generator=g) for _ in range(steps)]
    tgts = [torch.randint(0, cfg.vocab, (world, cfg.seq_len), generator=g) for _ in range(steps)]
    bad = []
    for s in range(steps):
        # same data every step for the last three so the loss visibly drops
        k = min(s, 3)
        l_sh = sharded.step(toks[k][rank:rank + 1].contiguous().pin_memory(), tgts[k][rank:rank + 1].contiguous().pin_memory())
        l_ref = single.step(toks[k].pin_memory(), tgts[k].pin_memory())
        parts = comm.host_all_gather(float(l_sh).hex().encode().ljust(32))
        mean = sum(float.fromhex(p.decode().strip()) for p in parts) / world
        if abs(mean - l_ref) > 0.03:
            bad.append((s, mean, l_ref))
        if rank == 0:
            print(f"step {s}: fsdp mean loss {mean:.4f}  single-rank loss {l_ref:.4f}", flush=True)
    # weights agree after training: compare this rank's shard of one layer with the single-rank copy
    u_sh, u_ref = sharded.layers[0], single.layers[0]
    lo = rank * u_sh.shard_numel
    n = min(u_sh.shard_numel, u_ref.shard_numel - lo)
    diff = (u_sh.master[:n] - u_ref.master[lo:lo + n]).abs().max().item() if n > 0 else 0.0
    if diff > 5e-3:
        bad.append(("weights", diff))
    err = comm.async_error()
    if err:
        bad.append(("async_error", err, comm.last_error()))
    flags = comm.host_all_gather(bytes([1 if bad else 0]))
    if bad:
        print(f"[rank {rank}] FSDP MISMATCH: {bad}", flush=True)
    elif rank == 0:
        norm = sharded.engine.last_grad_norm
        print(f"fsdp_worker OK on {world} ranks (max weight diff {diff:.2e}, fused_rs={fused}, sym_shards={sym}, clip={clip}"
              + (f", last gradient norm {float(norm):.4f}" if norm is not None else "") + ")", flush=True)
    torch.cuda.synchronize()
    comm.destroy()
    sys.exit(1 if any(f[0] for f in flags) else 0)


if __name__ == "__main__":
    main()
