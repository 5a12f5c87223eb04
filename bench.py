#!/usr/bin/env python
"""Headline benchmark: Llama-3-8B FSDP/ZeRO-3 training throughput (tokens/s) on N GPUs of one node.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One process per GPU. bf16 parameters with fp32 master weights and AdamW, sequence 4096,
micro-batch 1 per GPU, synthetic tokens (uniform over the vocabulary, seeded) and random-init
weights N(0, 0.02). Gradient reduce-scatters go through this package's communicator (one fused
reduce-scatter + cast + scale kernel per unit); parameter all-gathers are, between two GPUs, peer-to-peer
copies of the symmetric shards on the copy engines behind a barrier kernel of the communicator, and from
three GPUs up its zero-copy all-gather kernel (``--gather`` forces either). Two timed regions of K steps each, both bracketed by a barrier and a device
synchronisation and timed with CUDA events (max over ranks):

* ``value``  — steps fed from device-resident batches, loss left on the device;
* ``e2e``    — the public API call ``LlamaTrainer.step(tokens, targets)`` with the step's batch
               in pinned host memory (copied host->device inside the step) and the loss read
               back to the host every step.

Rank 0 prints one JSON line. On two or more GPUs the line also carries the collective stack's own headline, taken after
the timed regions: stock-NCCL time / this library's time per collective over a ladder of message sizes (``headline.
collectives_vs_nccl``) and, on 8 GPUs, the fused tensor-parallel and expert-parallel paths as fractions of their
rooflines (``headline.tp_roofline``, ``headline.ep_roofline``).

``--impl reference``: the reference project has no collective library that can be built for this GPU, so this arm runs
what its benchmark notes prescribe as the fallback, stock NCCL + cuBLAS on the same box: the same training job on
``torch.distributed.fsdp.fully_shard`` over the ``nccl`` backend (baseline/stock_torch_fsdp.py; nothing of this package
is imported there). ``vs_baseline`` of the normal line is ``value`` divided by that arm's number for the same N as
recorded in BASELINE_TOKENS_PER_S below.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading

METRIC = "llama3_8b_fsdp_train_tokens_per_sec"


# Stock torch FSDP on NCCL (``--impl reference``), tokens/s per N as measured on this pool's B200 boxes; None: not measured yet.
BASELINE_TOKENS_PER_S = {1: 13523.0, 2: 27459.0, 4: None, 8: 117010.0}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "power_w_max": max(power) if power else None, "samples": len(sm)}


def gpu_health(index: int):
    """NVLink error counters, ECC totals and the health verdict of the GPU the numbers were taken on (read-only, through
    NVML), recorded next to them; None when NVML cannot be read."""
    try:
        from rocm_systems_b200.tools.smi import Smi

        s = Smi()
        try:
            info, (level, reason) = s.info(index), s.health(index)
            return {"level": ("PASS", "WARN", "FAIL")[level] if 0 <= level <= 2 else str(level), "reason": reason, "nvlink_active": info["nvlinkActive"],
                    "nvlink_count": info["nvlinkCount"], "ecc_uncorrected": info["eccUncorrected"], "nvlink_errors": s.nvlink_errors(index)}
        finally:
            s.close()
    except Exception as e:  # noqa: BLE001 - an annotation must never fail the benchmark
        return {"unavailable": str(e)[:120]}


def take_headline(comm, trainer, dev, world: int) -> dict:
    """busbw against stock NCCL per collective, and on 8 GPUs the fused TP / EP paths against their rooflines. Runs after the
    timed regions, with the trainer's memory released first; a failure is recorded, it never fails the benchmark."""
    import gc

    import torch
    import torch.distributed as dist

    out = {}
    try:
        trainer.engine = None
        trainer.embed = trainer.layers = trainer.head = None
        gc.collect()
        torch.cuda.empty_cache()
        from rocm_systems_b200.bench import headline as hl

        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
        from rocm_systems_b200 import comm as bcomm

        alone = bcomm.init_from_env(device=dev.index, port_offset=29)   # a communicator with the library's default CTA budget
        out["collectives_vs_nccl"] = hl.collectives_vs_nccl(alone)
        if world == 8:
            out["tp_roofline"] = hl.tp_roofline(alone)
            out["ep_roofline"] = hl.ep_roofline(alone)
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
        alone.destroy()
    except Exception as e:  # noqa: BLE001
        out["error"] = f"{type(e).__name__}: {e}"[:300]
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3_8b", choices=["llama3_8b", "tiny"])
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (experiments; the headline uses the model's own)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--loss-curve", type=int, default=0, help="no timing: run this many steps from the initial weights and print every step's loss (both arms; for comparing their curves)")
    ap.add_argument("--lr", type=float, default=3e-4, help="AdamW learning rate of both arms (the headline uses the default)")
    ap.add_argument("--staged-shards", action="store_true",
                    help="keep parameter shards and gradient buffers in ordinary memory: the collectives then stage (default: symmetric memory, zero-copy)")
    ap.add_argument("--collectives", default="b200coll", choices=["b200coll", "nccl"],
                    help="nccl: the same trainer with stock NCCL collectives (control run; the metric name gets a _nccl_collectives suffix)")
    ap.add_argument("--gemm", default="own", choices=["own", "library"], help="linear layers on this package's tcgen05 kernel (default) or on cuBLAS")
    ap.add_argument("--gather", default="auto", choices=["auto", "kernel", "copy-engine"],
                    help="parameter all-gather by the copy engines (peer-to-peer copies behind a barrier kernel, no SM) or by this package's all-gather kernel; auto: copy engines between two GPUs, the kernel from three up")
    ap.add_argument("--no-overlap", action="store_true", help="run communication and optimizer on the compute stream (a sequential schedule, for checking)")
    ap.add_argument("--no-headline", action="store_true", help="skip the collective / fused-path summaries that follow the timed regions on 2+ GPUs")
    ap.add_argument("--reference-checkpointing", action="store_true", help="--impl reference: per-layer activation checkpointing from the start")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from baseline.stock_torch_fsdp import run as reference_run

        reference_run(args, ClockSampler)
        return

    import torch

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from rocm_systems_b200 import comm as bcomm
    from rocm_systems_b200.models.llama import LlamaConfig, LlamaTrainer
    from rocm_systems_b200.parallel.fsdp import AdamWConfig
    from rocm_systems_b200.ops import train_ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world != args.gpus and rank == 0:
        print(f"# note: --gpus {args.gpus} but WORLD_SIZE {world}; using WORLD_SIZE", file=sys.stderr)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if args.collectives == "nccl" and world > 1:
        import torch.distributed as dist

        from rocm_systems_b200.parallel.nccl_comm import NcclComm

        dist.init_process_group("nccl", device_id=dev)
        comm = NcclComm()
    else:
        # the training communicator's collectives overlap the GEMMs: 32 CTAs (the library's default, 64, is for collectives that run alone)
        comm = bcomm.init_from_env(device=local, max_ctas=32)

    from rocm_systems_b200.models import llama as llama_mod

    llama_mod.set_gemm(args.gemm)
    cfg = LlamaConfig.llama3_8b() if args.model == "llama3_8b" else LlamaConfig.tiny(512)
    if args.seq:
        cfg.seq_len = args.seq
    if args.layers:
        cfg.layers = args.layers
    trainer = LlamaTrainer(cfg, comm if world > 1 else None, dev, opt=AdamWConfig(lr=args.lr), fused_rs=args.collectives != "nccl", sym_shards=not args.staged_shards, overlap=not args.no_overlap,
                           copy_engine_gather={"auto": None, "kernel": False, "copy-engine": True}[args.gather])
    gather_mode = "none" if world == 1 else ("copy engines behind a barrier kernel" if trainer.engine.copy_engine_gather else "all-gather kernel of this package")
    S, B = cfg.seq_len, 1
    nbatches = 4
    g = torch.Generator().manual_seed(1234 + rank)
    host_tok = [torch.randint(0, cfg.vocab, (B, S), generator=g, dtype=torch.int64).pin_memory() for _ in range(nbatches)]
    host_tgt = [torch.randint(0, cfg.vocab, (B, S), generator=g, dtype=torch.int64).pin_memory() for _ in range(nbatches)]
    dev_tok = [t.to(dev) for t in host_tok]
    dev_tgt = [t.to(dev) for t in host_tgt]

    def sync_all() -> None:
        torch.cuda.synchronize()
        comm.host_barrier()
        torch.cuda.synchronize()

    if args.loss_curve:
        curve = [float(trainer.step(dev_tok[i % nbatches], dev_tgt[i % nbatches], return_loss=True)) for i in range(args.loss_curve)]
        if rank == 0:
            print(json.dumps({"impl": "ours", "n_gpus": world, "lr": args.lr, "layers": cfg.layers, "loss_curve": [round(x, 4) for x in curve]}))
        sync_all()
        comm.destroy()
        return

    for i in range(args.warmup):
        trainer.step(dev_tok[i % nbatches], dev_tgt[i % nbatches], return_loss=False)
    sync_all()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    def timed(fn) -> float:
        sync_all()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(args.steps):
            fn(i)
        b.record()
        sync_all()
        ms = a.elapsed_time(b)
        allms = comm.host_all_gather(float(ms).hex().encode().ljust(32))
        return max(float.fromhex(x.decode().strip()) for x in allms)

    l0, c0 = train_ops.LAUNCHES, bcomm.LAUNCHES
    ms_dev = timed(lambda i: trainer.step(dev_tok[i % nbatches], dev_tgt[i % nbatches], return_loss=False))
    launches = (train_ops.LAUNCHES - l0) + (bcomm.LAUNCHES - c0)
    losses = []
    ms_e2e = None
    if not args.no_e2e:
        ms_e2e = timed(lambda i: losses.append(trainer.step(host_tok[i % nbatches], host_tgt[i % nbatches], return_loss=True)))
    clocks = sampler.stop() if rank == 0 else {}

    tokens_per_step = world * B * S
    value = tokens_per_step * args.steps / (ms_dev / 1e3)
    base = BASELINE_TOKENS_PER_S.get(world) if args.model == "llama3_8b" and not args.seq and not args.layers else None
    peak_gb = trainer.memory_summary()["peak_gb"]
    headline = None
    if world > 1 and not args.no_headline and args.collectives == "b200coll":
        headline = take_headline(comm, trainer, dev, world)
    out = {
        "metric": METRIC + ("_nccl_collectives" if args.collectives == "nccl" else ""), "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": (value / base) if base else None, "dtype": "bf16",
        "data": "synthetic tokens uniform over the vocabulary (seeded), random-init weights N(0,0.02)",
        "config": {"model": "llama3-8b" if args.model == "llama3_8b" else "tiny", "global_batch": world * B, "seq_len": S,
                   "parallelism": f"fsdp{world}", "optimizer": "adamw fp32 master", "layers": cfg.layers, "hidden": cfg.hidden,
                   "linear_gemm": "tcgen05 cta-pair kernel of this package" if args.gemm == "own" else "cuBLAS",
                   "param_all_gather": gather_mode,
                   "l2": "working set per step (GBs of weights and activations) is far larger than the 126 MB L2; no flush needed"},
        "clocks": clocks, "gpu_launches": launches,
        "model_tflops_per_gpu": cfg.flops_per_token() * B * S / (ms_dev / args.steps / 1e3) / 1e12,
        "peak_mem_gb": peak_gb,
    }
    if base:
        out["baseline"] = {"what": "stock torch fully_shard on the nccl backend, same job, same pool (bench.py --impl reference)", "tokens_per_s": base}
    if headline is not None:
        out["headline"] = headline
    if ms_e2e is not None:
        out["e2e"] = {"value": tokens_per_step * args.steps / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * S * 8,
                      "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e / args.steps, "last_loss": losses[-1] if losses else None,
                      "losses": [round(float(x), 4) for x in losses]}
    if rank == 0:
        out["health"] = gpu_health(local)
        print(json.dumps(out))
    sync_all()
    comm.destroy()


if __name__ == "__main__":
    main()
