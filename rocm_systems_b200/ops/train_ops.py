"""Torch-facing wrappers of the hand-written training kernels (``csrc/fused/train_ops.cu``).

Each op calls the exported C symbol with raw device pointers on the current CUDA stream. There is
no eager-PyTorch fallback: on a machine with a GPU the kernels must be there, and a missing
library raises at import of :mod:`rocm_systems_b200._lib`.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib

LAUNCHES = 0  # kernels of this package launched through this module (bench.py reports it)

_sigs_done = False


def _lib_ops():
    global _sigs_done
    lib = _lib.load()
    if not _sigs_done:
        vp, ll, i32, f32 = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
        lib.b200ops_rmsnorm_fwd.argtypes = [vp, vp, vp, vp, ll, i32, f32, vp]
        lib.b200ops_rmsnorm_bwd.argtypes = [vp, vp, vp, vp, vp, vp, ll, i32, vp]
        lib.b200ops_rmsnorm_bwd_ctas.argtypes = [ll]
        lib.b200ops_rmsnorm_bwd_det.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, ll, i32, vp]
        lib.b200ops_adamw_bf16g.argtypes = [vp, vp, vp, vp, vp, ll, f32, f32, f32, f32, f32, i32, f32, vp]
        lib.b200ops_rope.argtypes = [vp, vp, ll, i32, i32, i32, i32, f32, vp]
        lib.b200ops_rope_oop.argtypes = [vp, vp, vp, ll, i32, i32, i32, i32, f32, vp]
        lib.b200ops_swiglu_fwd.argtypes = [vp, vp, ll, i32, vp]
        lib.b200ops_swiglu_bwd.argtypes = [vp, vp, vp, ll, i32, vp]
        lib.b200ops_cross_entropy.argtypes = [vp, vp, vp, ll, i32, ll, f32, vp]
        lib.b200ops_adamw.argtypes = [vp, vp, vp, vp, vp, ll, f32, f32, f32, f32, f32, i32, f32, vp]
        lib.b200ops_embedding_fwd.argtypes = [vp, vp, vp, ll, i32, vp]
        lib.b200ops_embedding_bwd.argtypes = [vp, vp, vp, ll, i32, vp]
        lib.b200ops_cast_scale.argtypes = [vp, vp, ll, f32, i32, vp]
        _sigs_done = True
    return lib


def _s() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ck(rc: int, what: str) -> None:
    global LAUNCHES
    if rc != 0:
        raise RuntimeError(f"{what}: CUDA error {rc}")
    LAUNCHES += 1


def _bf16c(t: torch.Tensor) -> torch.Tensor:
    assert t.is_cuda and t.dtype == torch.bfloat16, "bf16 CUDA tensor expected"
    return t if t.is_contiguous() else t.contiguous()


# ---- RMSNorm ---------------------------------------------------------------------------------------
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        x = _bf16c(x)
        H = x.shape[-1]
        T = x.numel() // H
        y = torch.empty_like(x)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        _ck(_lib_ops().b200ops_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), T, H, eps, _s()), "rmsnorm_fwd")
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dy = _bf16c(dy)
        H = x.shape[-1]
        T = x.numel() // H
        dx = torch.empty_like(x)
        lib = _lib_ops()
        # per-CTA partial sums of dw, added in a fixed order by a second small kernel: no atomics
        partials = torch.empty(int(lib.b200ops_rmsnorm_bwd_ctas(T)) * H, dtype=torch.float32, device=x.device)
        dw = torch.empty(H, dtype=w.dtype, device=x.device)
        assert w.dtype in (torch.bfloat16, torch.float32)
        _ck(lib.b200ops_rmsnorm_bwd_det(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), partials.data_ptr(), dw.data_ptr(),
                                        1 if w.dtype == torch.bfloat16 else 0, T, H, _s()), "rmsnorm_bwd")
        global LAUNCHES
        LAUNCHES += 1  # the column sum
        return dx, dw, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    return _RMSNorm.apply(x, w, eps)


# ---- rotary embedding ----------------------------------------------------------------------------------
def rope_table(seq_len: int, head_dim: int, theta: float, device) -> torch.Tensor:
    """[S, D/2, 2] float32 of (cos, sin) for positions 0..S-1 (rotate-half convention)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float64), inv)
    return torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.float32).to(device).contiguous()


class _Rope(torch.autograd.Function):
    """Rotates the first ``heads`` heads of each token row of ``qkv`` ([T, total_heads, D])."""

    @staticmethod
    def forward(ctx, qkv, table, heads):
        qkv = _bf16c(qkv)
        out = torch.empty_like(qkv)
        T, total, D = out.shape
        ctx.table, ctx.heads = table, heads
        _ck(_lib_ops().b200ops_rope_oop(qkv.data_ptr(), out.data_ptr(), table.data_ptr(), T, heads, total, D, table.shape[0], 1.0, _s()), "rope_fwd")
        return out

    @staticmethod
    def backward(ctx, g):
        g = _bf16c(g)  # the gradient is the inverse rotation
        out = torch.empty_like(g)
        T, total, D = g.shape
        _ck(_lib_ops().b200ops_rope_oop(g.data_ptr(), out.data_ptr(), ctx.table.data_ptr(), T, ctx.heads, total, D, ctx.table.shape[0], -1.0, _s()), "rope_bwd")
        return out, None, None


def rope_(qkv: torch.Tensor, table: torch.Tensor, heads: int) -> torch.Tensor:
    return _Rope.apply(qkv, table, heads)


# ---- SwiGLU -----------------------------------------------------------------------------------------------
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        gu = _bf16c(gu)
        F = gu.shape[-1] // 2
        T = gu.numel() // (2 * F)
        out = torch.empty(*gu.shape[:-1], F, dtype=gu.dtype, device=gu.device)
        _ck(_lib_ops().b200ops_swiglu_fwd(gu.data_ptr(), out.data_ptr(), T, F, _s()), "swiglu_fwd")
        ctx.save_for_backward(gu)
        return out

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        dout = _bf16c(dout)
        F = gu.shape[-1] // 2
        T = gu.numel() // (2 * F)
        dgu = torch.empty_like(gu)
        _ck(_lib_ops().b200ops_swiglu_bwd(gu.data_ptr(), dout.data_ptr(), dgu.data_ptr(), T, F, _s()), "swiglu_bwd")
        return dgu


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """``silu(gu[..., :F]) * gu[..., F:]`` for a fused gate/up projection output."""
    return _SwiGLU.apply(gu)


def swiglu_bwd(gu: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    """Gradient of :func:`swiglu` with respect to ``gu`` given the gradient of its output (no autograd graph: for
    callers that schedule their backward pass themselves)."""
    gu, dout = _bf16c(gu), _bf16c(dout)
    F = gu.shape[-1] // 2
    T = gu.numel() // (2 * F)
    assert dout.numel() == T * F
    dgu = torch.empty_like(gu)
    _ck(_lib_ops().b200ops_swiglu_bwd(gu.data_ptr(), dout.data_ptr(), dgu.data_ptr(), T, F, _s()), "swiglu_bwd")
    return dgu


# ---- loss, optimizer, embedding, casts (no autograd: the engine calls them explicitly) ---------------------
def cross_entropy_inplace(logits: torch.Tensor, targets: torch.Tensor, grad_scale: float) -> torch.Tensor:
    """Per-row loss of ``logits`` [T, V] (bf16); ``logits`` is overwritten with d(loss)/d(logits) * grad_scale."""
    assert logits.dtype == torch.bfloat16 and logits.dim() == 2 and logits.stride(1) == 1
    assert targets.dtype == torch.int64 and targets.is_contiguous()
    T, V = logits.shape
    loss = torch.empty(T, dtype=torch.float32, device=logits.device)
    _ck(_lib_ops().b200ops_cross_entropy(logits.data_ptr(), targets.data_ptr(), loss.data_ptr(), T, V, logits.stride(0), grad_scale, _s()), "cross_entropy")
    return loss


def adamw_(master, m, v, grad, param, lr, betas, eps, weight_decay, step, grad_scale=1.0) -> None:
    n = master.numel()
    assert m.numel() == n and v.numel() == n and grad.numel() == n and param.numel() == n
    assert master.dtype == torch.float32 and param.dtype == torch.bfloat16
    if grad.dtype == torch.bfloat16:  # straight from the backward pass: no fp32 copy of the gradient
        _ck(_lib_ops().b200ops_adamw_bf16g(master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(), param.data_ptr(), n, lr, betas[0], betas[1],
                                           eps, weight_decay, step, grad_scale, _s()), "adamw")
        return
    assert grad.dtype == torch.float32
    _ck(_lib_ops().b200ops_adamw(master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(), param.data_ptr(), n, lr, betas[0], betas[1], eps,
                                 weight_decay, step, grad_scale, _s()), "adamw")


def embedding(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    assert tokens.dtype == torch.int64 and table.dtype == torch.bfloat16 and table.is_contiguous()
    tokens = tokens.contiguous()
    H = table.shape[1]
    out = torch.empty(*tokens.shape, H, dtype=table.dtype, device=table.device)
    _ck(_lib_ops().b200ops_embedding_fwd(tokens.data_ptr(), table.data_ptr(), out.data_ptr(), tokens.numel(), H, _s()), "embedding_fwd")
    return out


def embedding_bwd_(tokens: torch.Tensor, dout: torch.Tensor, dtable_f32: torch.Tensor) -> None:
    dout = _bf16c(dout)
    H = dtable_f32.shape[1]
    _ck(_lib_ops().b200ops_embedding_bwd(tokens.contiguous().data_ptr(), dout.data_ptr(), dtable_f32.data_ptr(), tokens.numel(), H, _s()), "embedding_bwd")


def cast_scale_(src_bf16: torch.Tensor, dst_f32: torch.Tensor, scale: float, accumulate: bool = False) -> None:
    assert src_bf16.numel() == dst_f32.numel() and src_bf16.is_contiguous() and dst_f32.is_contiguous()
    _ck(_lib_ops().b200ops_cast_scale(src_bf16.data_ptr(), dst_f32.data_ptr(), src_bf16.numel(), scale, int(accumulate), _s()), "cast_scale")


def gemm_bf16_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None, bn: int = 0, max_ctas: int = 0) -> torch.Tensor:
    """``a @ b.T`` for bf16 row-major ``a`` [M, K] and ``b`` [N, K] on the hand-written tcgen05
    kernel (TMA-fed, accumulators in tensor memory). Library GEMMs are not used on this path."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1 and a.shape[1] == b.shape[1]
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    lib = _lib_ops()
    if not hasattr(lib, "_gemm_sig"):
        vp, i32 = ctypes.c_void_p, ctypes.c_int
        lib.b200ops_gemm_bf16_tn.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp]
        lib._gemm_sig = True
    _ck(lib.b200ops_gemm_bf16_tn(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0), bn, max_ctas, _s()), "gemm_bf16_tn")
    return out


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None, bn: int = 0, max_ctas: int = 0) -> torch.Tensor:
    """``a @ b.T`` in bf16 with fp32 accumulation on the CTA-pair tcgen05 kernel (csrc/fused/gemm_pair_sm100.cuh).

    ``a`` is [M, K] and ``b`` [N, K] as tensors; each may be a row-major matrix or the transposed view of one
    (``x.t()``): the kernel reads either memory order directly (K-major or MN-major operand), so the three GEMMs of a
    linear layer need no transposed copy:

        y  = gemm(x, w)              # x [T, K], w [N, K]
        dx = gemm(dy, w.t())         # dy [T, N], w.t() [K, N]
        dw = gemm(dy.t(), x.t())     # dy.t() [N, T], x.t() [K, T]

    ``out`` ([M, N], unit column stride) may be a view into a larger buffer."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1]
    M, K = a.shape
    N = b.shape[0]

    def major(t):  # (stored with the row index contiguous?, leading dimension)
        if t.stride(1) == 1:
            return 0, t.stride(0)
        assert t.stride(0) == 1, "operand must be a row-major matrix or the transpose of one"
        return 1, t.stride(1)

    a_mn, lda = major(a)
    b_mn, ldb = major(b)
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    assert out.dtype == torch.bfloat16 and out.shape == (M, N) and out.stride(1) == 1
    lib = _lib_ops()
    if not hasattr(lib, "_gemm_pair_sig"):
        vp, i32 = ctypes.c_void_p, ctypes.c_int
        lib.b200ops_gemm_bf16_pair.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp]
        lib._gemm_pair_sig = True
    _ck(lib.b200ops_gemm_bf16_pair(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, lda, ldb, out.stride(0), a_mn, b_mn, bn, max_ctas, _s()), "gemm_bf16_pair")
    return out


def gemm_take_error() -> int:
    """Code of the first bounded wait that gave up inside a tcgen05 kernel (0: none); synchronises."""
    return int(_lib_ops().b200ops_gemm_take_error())
