"""Block-scaled fp8 (e4m3) linear algebra: quantisers and the tcgen05 GEMM behind them
(csrc/fused/gemm_fp8_sm100.cu), with plain PyTorch statements of the same arithmetic as oracles.

Layout contract (what the kernel reads):

* activations ``x`` [M, K]  ->  ``q`` [M, K] e4m3 and ``s`` [K / 128, M] fp32, one scale per row and 128 channels,
  ``scale = max(amax, 1e-10) * fp32(1 / 448)`` and ``q = x / scale`` (an IEEE division), so the kernels and these oracles agree bit for bit;
* weights ``w`` [N, K]  ->  ``q`` [N, K] e4m3 and ``s`` [ceil(N / 128), K / 128] fp32, one scale per 128 x 128 block;
* ``gemm(xq, xs, wq, ws)[m, n] = sum_kb xs[kb, m] * ws[n // 128, kb] * dot(xq[m, kb], wq[n, kb])`` with fp32 accumulation,
  rounded to bf16 once at the end.

The reference stack has no fp8 GEMM; its benchmark harness only carries fp8 as a datatype of the collectives
(rccl-tests src/rccl_float8.h:63-245).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import train_ops

E4M3_MAX = 448.0


# ---- oracles: run anywhere -------------------------------------------------------------------------------------
def ref_quantize_act(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    M, K = x.shape
    assert K % 128 == 0
    g = x.float().view(M, K // 128, 128)
    scale = g.abs().amax(-1).clamp_min(1e-10) * (1.0 / E4M3_MAX)  # [M, K/128]
    q = (g / scale.unsqueeze(-1)).to(torch.float8_e4m3fn).view(M, K)
    return q, scale.t().contiguous()                                # scales block-major: [K/128, M]


def ref_quantize_weight(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    N, K = w.shape
    assert K % 128 == 0
    nb = (N + 127) // 128
    pad = torch.zeros(nb * 128, K, dtype=torch.float32, device=w.device)
    pad[:N] = w.float()
    blocks = pad.view(nb, 128, K // 128, 128)
    scale = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-10) * (1.0 / E4M3_MAX)   # [nb, K/128]
    q = (blocks / scale[:, None, :, None]).to(torch.float8_e4m3fn).view(nb * 128, K)[:N].contiguous()
    return q, scale.contiguous()


def ref_dequantize_act(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    M, K = q.shape
    return (q.float().view(M, K // 128, 128) * s.t().unsqueeze(-1)).view(M, K)


def ref_dequantize_weight(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    N, K = q.shape
    rows = torch.arange(N, device=q.device) // 128
    return (q.float().view(N, K // 128, 128) * s[rows].unsqueeze(-1)).view(N, K)


def ref_gemm(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Block by block, as the kernel accumulates: fp32 partial products scaled and summed in K order.
    ``out_dtype=torch.float32`` returns the accumulator before the final rounding (what a fused epilogue sees)."""
    M, K = xq.shape
    N = wq.shape[0]
    rows = torch.arange(N, device=wq.device) // 128
    out = torch.zeros(M, N, dtype=torch.float32, device=xq.device)
    for kb in range(K // 128):
        part = xq[:, kb * 128:(kb + 1) * 128].float() @ wq[:, kb * 128:(kb + 1) * 128].float().t()
        out += part * xs[kb].unsqueeze(1) * ws[rows, kb].unsqueeze(0)
    return out.to(out_dtype)


# ---- the kernels ---------------------------------------------------------------------------------------------------
def _lib():
    lib = train_ops._lib_ops()
    if not hasattr(lib, "_fp8_sig"):
        vp, i32 = ctypes.c_void_p, ctypes.c_int
        lib.b200ops_quant_e4m3_1x128.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp]
        lib.b200ops_quant_e4m3_1x128_strided.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, vp]
        lib.b200ops_quant_e4m3_128x128.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp]
        lib.b200ops_gemm_fp8_block_tn.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp]
        lib._fp8_sig = True
    return lib


def quantize_act(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 128 == 0
    M, K = x.shape
    q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(K // 128, M, dtype=torch.float32, device=x.device)
    train_ops._ck(_lib().b200ops_quant_e4m3_1x128(x.data_ptr(), q.data_ptr(), s.data_ptr(), M, K, x.stride(0), q.stride(0), train_ops._s()), "quant_e4m3_1x128")
    return q, s


def quantize_act_into(x: torch.Tensor, q: torch.Tensor, s: torch.Tensor, row0: int) -> None:
    """Quantise ``x`` [m, K] into rows ``row0 .. row0 + m`` of a larger ``q`` [M, K] and the matching columns of its scale
    table ``s`` [K / 128, M] (a rank filling its shard of a gathered activation)."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and x.shape[1] % 128 == 0
    m, K = x.shape
    M = q.shape[0]
    assert q.dtype == torch.float8_e4m3fn and q.shape[1] == K and q.stride(1) == 1 and 0 <= row0 and row0 + m <= M
    assert s.dtype == torch.float32 and tuple(s.shape) == (K // 128, M) and s.is_contiguous()
    train_ops._ck(_lib().b200ops_quant_e4m3_1x128_strided(x.data_ptr(), q.data_ptr() + row0 * q.stride(0), s.data_ptr() + 4 * row0, m, K, x.stride(0), q.stride(0),
                                                          M, train_ops._s()), "quant_e4m3_1x128_strided")


def quantize_weight(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    assert w.is_cuda and w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1 and w.shape[1] % 128 == 0
    N, K = w.shape
    q = torch.empty(N, K, dtype=torch.float8_e4m3fn, device=w.device)
    s = torch.empty((N + 127) // 128, K // 128, dtype=torch.float32, device=w.device)
    train_ops._ck(_lib().b200ops_quant_e4m3_128x128(w.data_ptr(), q.data_ptr(), s.data_ptr(), N, K, w.stride(0), q.stride(0), train_ops._s()), "quant_e4m3_128x128")
    return q, s


def gemm(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, out: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
    """``dequant(xq, xs) @ dequant(wq, ws).T`` in bf16 on the block-scaled tcgen05 kernel."""
    assert xq.is_cuda and xq.dtype == torch.float8_e4m3fn and wq.dtype == torch.float8_e4m3fn
    assert xq.stride(1) == 1 and wq.stride(1) == 1 and xq.shape[1] == wq.shape[1]
    M, K = xq.shape
    N = wq.shape[0]
    assert tuple(xs.shape) == (K // 128, M) and tuple(ws.shape) == ((N + 127) // 128, K // 128) and xs.is_contiguous() and ws.is_contiguous()
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=xq.device)
    train_ops._ck(_lib().b200ops_gemm_fp8_block_tn(xq.data_ptr(), xs.data_ptr(), wq.data_ptr(), ws.data_ptr(), out.data_ptr(), M, N, K, xq.stride(0), wq.stride(0),
                                                   out.stride(0), max_ctas, train_ops._s()), "gemm_fp8_block_tn")
    return out


def linear(x: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` for bf16 ``x`` against a weight quantised once with ``quantize_weight``."""
    xq, xs = quantize_act(x)
    return gemm(xq, xs, wq, ws)
