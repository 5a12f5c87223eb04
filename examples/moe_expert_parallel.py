"""A mixture-of-experts layer with the experts spread over the ranks: routing, fp8 dispatch into the
experts' ranks, grouped expert GEMMs and the gate-weighted combine, compared with a plain PyTorch layer.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/moe_expert_parallel.py
"""
import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from rocm_systems_b200.comm import init_from_env  # noqa: E402
from rocm_systems_b200.ops import train_ops  # noqa: E402
from rocm_systems_b200.parallel.ep import MoELayer  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=256, help="experts over all ranks")
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=1024)
    ap.add_argument("--tokens", type=int, default=2048, help="tokens per rank")
    ap.add_argument("--fp8-experts", action="store_true", help="run the gate/up expert GEMM on the fp8 rows as they arrived (block-quantised weights)")
    ap.add_argument("--backward", action="store_true", help="also time forward + backward (token, router-logit and expert-weight gradients); bf16 experts only")
    a = ap.parse_args()
    comm = init_from_env()
    moe = MoELayer(comm, a.experts // comm.nranks, a.hidden, a.ffn, a.topk, a.tokens, seed=5, fp8_experts=a.fp8_experts)
    x = torch.randn(a.tokens, a.hidden, device=comm.device).to(torch.bfloat16)
    logits = torch.randn(a.tokens, moe.E, device=comm.device)
    want = moe.reference_forward(x, logits).float()
    got = moe.forward(x, logits).float()
    torch.cuda.synchronize()
    code = train_ops.gemm_take_error()
    err, scale = float((got - want).abs().max()), float(want.abs().max())
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(2):
        moe.forward(x, logits)
    torch.cuda.synchronize()
    comm.host_barrier()
    start.record()
    for _ in range(5):
        moe.forward(x, logits)
    stop.record()
    torch.cuda.synchronize()
    if comm.rank == 0:
        print(f"EP={comm.nranks} experts {moe.E} top-{a.topk} tokens/rank {a.tokens}: max |error| {err:.3e} (output scale {scale:.3e}), "
              f"{start.elapsed_time(stop) / 5:.3f} ms per layer, kernel status {code}", flush=True)
    ok = code == 0 and err <= 6e-2 * scale + 1e-3  # activations cross the wire as fp8 e4m3 with one scale per 128 channels
    if a.backward and not a.fp8_experts:
        dy = torch.randn(a.tokens, a.hidden, device=comm.device).to(torch.bfloat16)
        for _ in range(2):
            moe.forward(x, logits)
            moe.backward(dy)
        torch.cuda.synchronize()
        comm.host_barrier()
        start.record()
        for _ in range(5):
            moe.forward(x, logits)
            dx, dlogits = moe.backward(dy)
        stop.record()
        torch.cuda.synchronize()
        bcode = train_ops.gemm_take_error()
        if comm.rank == 0:
            print(f"forward + backward: {start.elapsed_time(stop) / 5:.3f} ms; dx {tuple(dx.shape)}, d_logits {tuple(dlogits.shape)}, "
                  f"grads {', '.join(f'{k} {tuple(v.shape)}' for k, v in moe.grads.items())}, kernel status {bcode}", flush=True)
        ok = ok and bcode == 0
    moe.free()
    comm.destroy()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
