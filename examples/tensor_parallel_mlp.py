"""Tensor-parallel SwiGLU MLP with sequence-parallel activations, run through the two fused kernels
(all-gather -> GEMM + SwiGLU, GEMM -> reduce-scatter) and compared with the unfused composition.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/tensor_parallel_mlp.py

Each rank holds `rows` tokens, a [2 * ffn / world, hidden] slice of the gate/up projection and a
[hidden, ffn / world] slice of the down projection; the output comes back token-sharded.
"""
import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from rocm_systems_b200.comm import init_from_env  # noqa: E402
from rocm_systems_b200.ops import train_ops  # noqa: E402
from rocm_systems_b200.parallel.tp import TensorParallelAttention, TensorParallelMLP, TensorParallelMLPFp8  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=1024, help="tokens per rank")
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672, help="whole intermediate size")
    ap.add_argument("--fp8", action="store_true", help="block-scaled e4m3 operands: half the all-gather bytes, fp8 tensor-core rate; "
                    "compared with the PyTorch statement of the same quantised arithmetic")
    ap.add_argument("--backward", action="store_true", help="also time forward + backward (the same two fused kernels on transposed weights, "
                    "weight gradients as local GEMMs); bf16 form only")
    ap.add_argument("--attention", action="store_true", help="also run the tensor-parallel attention half of the layer")
    ap.add_argument("--heads", type=int, default=64)
    ap.add_argument("--kv-heads", type=int, default=8)
    a = ap.parse_args()
    comm = init_from_env()
    mlp = (TensorParallelMLPFp8 if a.fp8 else TensorParallelMLP)(comm, a.rows, a.hidden, a.ffn // comm.nranks, comm.device, seed=1)
    x = (torch.randn(a.rows, a.hidden, device=comm.device) * 0.5).to(torch.bfloat16)
    want = mlp.reference_forward(x).float()
    got = mlp.forward(x).float()
    torch.cuda.synchronize()
    err, scale = float((got - want).abs().max()), float(want.abs().max())
    code = train_ops.gemm_take_error()  # non-zero if a bounded wait inside the kernels ran out
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        mlp.forward(x)
    torch.cuda.synchronize()
    comm.host_barrier()
    start.record()
    for _ in range(10):
        mlp.forward(x)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / 10
    flops = 2.0 * a.rows * comm.nranks * a.hidden * (3 * a.ffn // comm.nranks)
    if comm.rank == 0:
        print(f"{'fp8 ' if a.fp8 else ''}TP={comm.nranks} tokens {a.rows * comm.nranks} hidden {a.hidden} ffn {a.ffn}: max |error| {err:.3e} (output scale {scale:.3e}), "
              f"{ms:.3f} ms per layer, {flops / ms / 1e9:.0f} TFLOP/s per GPU, kernel status {code}", flush=True)
    ok = code == 0 and err <= 3e-2 * scale + 1e-3
    if a.backward and not a.fp8:
        dy = (torch.randn(a.rows, a.hidden, device=comm.device) * 0.5).to(torch.bfloat16)
        for _ in range(3):
            mlp.forward(x)
            mlp.backward(dy)
        torch.cuda.synchronize()
        comm.host_barrier()
        start.record()
        for _ in range(10):
            mlp.forward(x)
            dx = mlp.backward(dy)
        stop.record()
        torch.cuda.synchronize()
        bms = start.elapsed_time(stop) / 10
        bcode = train_ops.gemm_take_error()
        if comm.rank == 0:
            print(f"forward + backward: {bms:.3f} ms, {3 * flops / bms / 1e9:.0f} TFLOP/s per GPU of model FLOPs; dx {tuple(dx.shape)}, "
                  f"grads {', '.join(f'{k} {tuple(v.shape)}' for k, v in mlp.grads.items())}, kernel status {bcode}", flush=True)
        ok = ok and bcode == 0
    mlp.free()
    if a.attention:
        # The other half of the layer on the same two kernels: QKV projection inside the all-gather, output projection
        # inside the reduce-scatter, this rank's heads attended locally.
        seq = min(4096, a.rows * comm.nranks)
        att = TensorParallelAttention(comm, a.rows, a.hidden, a.heads, a.kv_heads, seq, comm.device, seed=2)
        want = att.reference_forward(x).float()
        got = att.forward(x).float()
        torch.cuda.synchronize()
        aerr, ascale = float((got - want).abs().max()), float(want.abs().max())
        acode = train_ops.gemm_take_error()
        if comm.rank == 0:
            print(f"attention: {a.heads} heads ({a.kv_heads} kv) over TP={comm.nranks}, sequences of {seq}: max |error| {aerr:.3e} (output scale {ascale:.3e}), "
                  f"kernel status {acode}", flush=True)
        ok = ok and acode == 0 and aerr <= 3e-2 * ascale + 1e-3
        att.free()
    comm.destroy()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
