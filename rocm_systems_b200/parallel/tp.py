"""Tensor-parallel (with sequence-parallel activations) MLP on the fused kernels.

``TensorParallelMLP`` holds this rank's shards of a SwiGLU MLP: ``w13`` (gate and up rows of its
1/N of the hidden features, interleaved per 256-row tile as the fused kernel wants) and ``w2`` (the
matching K-shard). ``forward`` takes this rank's rows of the activations and returns this rank's
rows of the output:

    all-gather(x) -> x @ w13^T -> SwiGLU -> @ w2^T -> reduce-scatter

as two kernels, ``b200collAgGemm`` and ``b200collGemmRs`` (csrc/fused/tp_fused.cu), each of which
moves its data over NVLink from inside the tcgen05 GEMM. ``reference_forward`` is the unfused
composition (collectives of this package + library GEMMs) used as oracle and timing baseline.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _lib
from ..ops import train_ops

_done = False


def _lib_tp():
    global _done
    lib = _lib.load()
    if not _done:
        vp, i32 = ctypes.c_void_p, ctypes.c_int
        lib.b200collAgGemm.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]
        lib.b200collGemmRs.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, vp]
        lib.b200collGemmRsWorkspaceBytes.argtypes = [i32, i32, i32]
        lib.b200collGemmRsWorkspaceBytes.restype = ctypes.c_size_t
        lib.b200collAgGemmFp8.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]
        lib.b200collGemmRsFp8.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp]
        _done = True
    return lib


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor, tile: int = 256) -> torch.Tensor:
    """Stack gate and up rows so that every ``tile`` rows hold tile/2 gate rows then the tile/2 up
    rows of the same output features (the layout the fused SwiGLU epilogue reads)."""
    F, K = w_gate.shape
    h = tile // 2
    assert F % h == 0
    g = w_gate.view(F // h, h, K)
    u = w_up.view(F // h, h, K)
    return torch.stack([g, u], dim=1).reshape(2 * F, K).contiguous()


def deinterleave_gate_up(w13: torch.Tensor, tile: int = 256):
    """Inverse of :func:`interleave_gate_up`: (gate rows, up rows)."""
    F2, K = w13.shape
    h = tile // 2
    v = w13.view(F2 // tile, 2, h, K)
    return v[:, 0].reshape(F2 // 2, K), v[:, 1].reshape(F2 // 2, K)


class TensorParallelMLP:
    """The MLP half of a tensor-parallel transformer layer with sequence-parallel activations: gate and up projections
    (column-parallel, interleaved per tile) inside the all-gather with the SwiGLU in the epilogue, down projection
    (row-parallel) inside the reduce-scatter. ``backward`` runs the same two fused kernels on the transposed weights
    (the gradient of a reduce-scatter is an all-gather and the other way round) and leaves the weight gradients of this
    rank's shards in ``grads``; weights are random.
    """

    def __init__(self, comm, rows_per_rank: int, hidden: int, ffn_local: int, device=None, std: float = 0.02, seed: int = 0,
                 comm_ctas: int = 0):
        self.comm = comm
        self.n, self.rank = comm.nranks, comm.rank
        self.rows, self.hidden, self.f = rows_per_rank, hidden, ffn_local
        self.device = device or comm.device
        self.comm_ctas = comm_ctas
        g = torch.Generator(device=self.device).manual_seed(seed + 7919 * self.rank)
        wg = (torch.randn(ffn_local, hidden, device=self.device, generator=g) * std).to(torch.bfloat16)
        wu = (torch.randn(ffn_local, hidden, device=self.device, generator=g) * std).to(torch.bfloat16)
        self.w_gate, self.w_up = wg, wu
        self.tile = 256 if (2 * ffn_local) % 256 == 0 else 128
        self.w13 = interleave_gate_up(wg, wu, self.tile)
        self.w2 = (torch.randn(hidden, ffn_local, device=self.device, generator=g) * std).to(torch.bfloat16)
        M = self.n * rows_per_rank
        lib = _lib_tp()
        self._x_sym = comm.sym_alloc(M * hidden * 2)
        self.x_full = self._x_sym.tensor((M, hidden), torch.bfloat16)
        self._ws = comm.sym_alloc(int(lib.b200collGemmRsWorkspaceBytes(rows_per_rank, hidden, self.n)))
        self.act = torch.empty(M, ffn_local, dtype=torch.bfloat16, device=self.device)
        self.y = torch.empty(rows_per_rank, hidden, dtype=torch.bfloat16, device=self.device)
        self._dy_sym = self._ws_b = None          # backward buffers, made by the first backward()
        self._w2_t = self._w13_t = None           # transposed weights (the fused kernels read B with the reduction index contiguous)
        self.grads: dict = {}

    def my_rows(self) -> torch.Tensor:
        """Where this rank writes its rows of the activations before ``forward``."""
        return self.x_full[self.rank * self.rows:(self.rank + 1) * self.rows]

    def weights_changed(self) -> None:
        """Call after ``w13`` or ``w2`` was updated in place: the transposed copies used by ``backward`` are rebuilt."""
        self._w2_t = self._w13_t = None
        self.w_gate, self.w_up = deinterleave_gate_up(self.w13, self.tile)

    def backward(self, dy_local: torch.Tensor) -> torch.Tensor:
        """Gradients of the latest ``forward`` (its gathered input rows and its ``act`` must still be in place), on the
        current stream.

            d_act = all-gather(dy) @ w2          one fused kernel (all-gather -> GEMM); also leaves dy of all tokens here
            gate/up pre-activations              recomputed from the gathered input with a local GEMM (not kept by forward)
            d_gu  = SwiGLU'(gu) * d_act          element-wise, in the per-tile interleaved layout of w13
            dx    = reduce-scatter(d_gu @ w13)   one fused kernel (GEMM -> reduce-scatter)
            dw2   = dy^T @ act,  dw13 = d_gu^T @ x     local GEMMs over all tokens: this rank owns these shards alone

        Returns this rank's rows of dx; ``grads["w13"]`` (interleaved like ``w13``) and ``grads["w2"]`` hold the weight gradients."""
        lib = _lib_tp()
        s = torch.cuda.current_stream().cuda_stream
        M = self.n * self.rows
        if self._dy_sym is None:
            self._dy_sym = self.comm.sym_alloc(M * self.hidden * 2)
            self.dy_full = self._dy_sym.tensor((M, self.hidden), torch.bfloat16)
            self._ws_b = self.comm.sym_alloc(int(lib.b200collGemmRsWorkspaceBytes(self.rows, self.hidden, self.n)))
            self.dact = torch.empty(M, self.f, dtype=torch.bfloat16, device=self.device)
            self.dx = torch.empty(self.rows, self.hidden, dtype=torch.bfloat16, device=self.device)
        if self._w2_t is None:
            self._w2_t = self.w2.t().contiguous()      # [ffn_local, hidden]
            self._w13_t = self.w13.t().contiguous()    # [hidden, 2 ffn_local]
        self.dy_full[self.rank * self.rows:(self.rank + 1) * self.rows].copy_(dy_local)
        _lib.check(lib.b200collAgGemm(self.comm.handle, self.dy_full.data_ptr(), self._w2_t.data_ptr(), self.dact.data_ptr(), self.rows, self.f,
                                      self.hidden, 0, self.comm_ctas, s), "b200collAgGemm (backward)")
        gu = train_ops.gemm(self.x_full, self.w13)                                  # [M, 2 ffn_local], gate and up interleaved per tile
        nt = 2 * self.f // self.tile
        dgu = train_ops.swiglu_bwd(gu.view(M * nt, self.tile), self.dact.view(M * nt, self.tile // 2)).view(M, 2 * self.f)
        _lib.check(lib.b200collGemmRs(self.comm.handle, dgu.data_ptr(), self._w13_t.data_ptr(), self._ws_b.ptr, self.dx.data_ptr(), self.rows,
                                      self.hidden, 2 * self.f, s), "b200collGemmRs (backward)")
        train_ops.LAUNCHES += 2
        self.grads["w2"] = train_ops.gemm(self.dy_full.t(), self.act.t())           # [hidden, ffn_local]
        self.grads["w13"] = train_ops.gemm(dgu.t(), self.x_full.t())                # [2 ffn_local, hidden]
        return self.dx

    def ag_gemm(self, stream=None) -> torch.Tensor:
        """all-gather(x) @ w13^T with SwiGLU: ``act`` [M, ffn_local]. This rank's rows must be in ``my_rows()``."""
        s = (stream or torch.cuda.current_stream()).cuda_stream
        _lib.check(_lib_tp().b200collAgGemm(self.comm.handle, self.x_full.data_ptr(), self.w13.data_ptr(), self.act.data_ptr(), self.rows,
                                            2 * self.f, self.hidden, 1, self.comm_ctas, s), "b200collAgGemm")
        train_ops.LAUNCHES += 1
        return self.act

    def gemm_rs(self, stream=None) -> torch.Tensor:
        """reduce-scatter(act @ w2^T): this rank's rows of the output."""
        s = (stream or torch.cuda.current_stream()).cuda_stream
        _lib.check(_lib_tp().b200collGemmRs(self.comm.handle, self.act.data_ptr(), self.w2.data_ptr(), self._ws.ptr, self.y.data_ptr(), self.rows,
                                            self.hidden, self.f, s), "b200collGemmRs")
        train_ops.LAUNCHES += 1
        return self.y

    def forward(self, x_local: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        if x_local is not None:
            self.my_rows().copy_(x_local)
        self.ag_gemm(stream)
        return self.gemm_rs(stream)

    def reference_forward(self, x_local: torch.Tensor) -> torch.Tensor:
        """Unfused: all_gather, two library GEMMs, SwiGLU, reduce_scatter."""
        M = self.n * self.rows
        xg = torch.empty(M, self.hidden, dtype=torch.bfloat16, device=self.device)
        self.comm.all_gather(x_local.contiguous(), xg)
        g = xg @ self.w_gate.t()
        u = xg @ self.w_up.t()
        a = (torch.nn.functional.silu(g.float()) * u.float()).to(torch.bfloat16)
        part = a @ self.w2.t()
        out = torch.empty(self.rows, self.hidden, dtype=torch.bfloat16, device=self.device)
        self.comm.reduce_scatter(part, out)
        return out

    def free(self) -> None:
        torch.cuda.synchronize()
        self._x_sym.free()
        self._ws.free()
        if self._dy_sym is not None:
            self._dy_sym.free()
            self._ws_b.free()


def fp8_mlp_partial_oracle(x_full: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """What one rank of :class:`TensorParallelMLPFp8` contributes, in plain PyTorch with the kernels' arithmetic: the
    gathered activations and the interleaved gate/up weight quantised block-wise to e4m3, fp32 accumulation, SwiGLU on the
    fp32 accumulators, bf16 activations quantised again for the down projection, and the partial result rounded to bf16
    (the form in which partials cross NVLink). Returns [M, hidden] bf16. Runs on any device."""
    from ..ops import fp8
    M = x_full.shape[0]
    F = w_gate.shape[0]
    xq, xs = fp8.ref_quantize_act(x_full)
    wq, ws = fp8.ref_quantize_weight(interleave_gate_up(w_gate, w_up, 128))
    h = fp8.ref_gemm(xq, xs, wq, ws, out_dtype=torch.float32).view(M, F // 64, 2, 64)
    act = (torch.nn.functional.silu(h[:, :, 0]) * h[:, :, 1]).reshape(M, F).to(torch.bfloat16)
    aq, a_s = fp8.ref_quantize_act(act)
    w2q, w2s = fp8.ref_quantize_weight(w2)
    return fp8.ref_gemm(aq, a_s, w2q, w2s)


class TensorParallelMLPFp8:
    """:class:`TensorParallelMLP` on block-scaled fp8 operands (``b200collAgGemmFp8`` / ``b200collGemmRsFp8``,
    csrc/fused/tp_fused_fp8.cu). Each rank quantises its own rows (e4m3 + one scale per row and 128 channels) straight into
    the symmetric buffers, so the all-gather moves half the bytes of the bf16 form; weights are quantised once per
    128 x 128 block. ``hidden`` and ``ffn_local`` are multiples of 128.
    """

    def __init__(self, comm, rows_per_rank: int, hidden: int, ffn_local: int, device=None, std: float = 0.02, seed: int = 0,
                 comm_ctas: int = 0):
        from ..ops import fp8
        assert hidden % 128 == 0 and ffn_local % 128 == 0
        self.comm = comm
        self.n, self.rank = comm.nranks, comm.rank
        self.rows, self.hidden, self.f = rows_per_rank, hidden, ffn_local
        self.device = device or comm.device
        self.comm_ctas = comm_ctas
        g = torch.Generator(device=self.device).manual_seed(seed + 7919 * self.rank)
        self.w_gate = (torch.randn(ffn_local, hidden, device=self.device, generator=g) * std).to(torch.bfloat16)
        self.w_up = (torch.randn(ffn_local, hidden, device=self.device, generator=g) * std).to(torch.bfloat16)
        self.w2 = (torch.randn(hidden, ffn_local, device=self.device, generator=g) * std).to(torch.bfloat16)
        self.w13_q, self.w13_s = fp8.quantize_weight(interleave_gate_up(self.w_gate, self.w_up, 128))
        self.w2_q, self.w2_s = fp8.quantize_weight(self.w2)
        M = self.M = self.n * rows_per_rank
        lib = _lib_tp()
        self._x_sym = comm.sym_alloc(M * hidden)
        self._s_sym = comm.sym_alloc((hidden // 128) * M * 4)
        self.x_q = self._x_sym.tensor((M, hidden), torch.float8_e4m3fn)
        self.x_s = self._s_sym.tensor((hidden // 128, M), torch.float32)
        self._ws = comm.sym_alloc(int(lib.b200collGemmRsWorkspaceBytes(rows_per_rank, hidden, self.n)))
        self.act = torch.empty(M, ffn_local, dtype=torch.bfloat16, device=self.device)
        self.y = torch.empty(rows_per_rank, hidden, dtype=torch.bfloat16, device=self.device)

    def set_rows(self, x_local: torch.Tensor) -> None:
        """Quantise this rank's rows of the activations into its shard of the gathered buffers."""
        from ..ops import fp8
        fp8.quantize_act_into(x_local, self.x_q, self.x_s, self.rank * self.rows)
        train_ops.LAUNCHES += 1

    def ag_gemm(self, stream=None) -> torch.Tensor:
        s = (stream or torch.cuda.current_stream()).cuda_stream
        _lib.check(_lib_tp().b200collAgGemmFp8(self.comm.handle, self.x_q.data_ptr(), self.x_s.data_ptr(), self.w13_q.data_ptr(), self.w13_s.data_ptr(),
                                               self.act.data_ptr(), self.rows, 2 * self.f, self.hidden, 1, self.comm_ctas, s), "b200collAgGemmFp8")
        train_ops.LAUNCHES += 1
        return self.act

    def gemm_rs(self, stream=None) -> torch.Tensor:
        from ..ops import fp8
        st = stream or torch.cuda.current_stream()
        with torch.cuda.stream(st):      # the quantiser and its temporaries live on the stream of the kernel that reads them
            aq, a_s = fp8.quantize_act(self.act)
            _lib.check(_lib_tp().b200collGemmRsFp8(self.comm.handle, aq.data_ptr(), a_s.data_ptr(), self.w2_q.data_ptr(), self.w2_s.data_ptr(), self._ws.ptr,
                                                   self.y.data_ptr(), self.rows, self.hidden, self.f, st.cuda_stream), "b200collGemmRsFp8")
        train_ops.LAUNCHES += 2
        return self.y

    def forward(self, x_local: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        if x_local is not None:
            with torch.cuda.stream(stream or torch.cuda.current_stream()):
                self.set_rows(x_local)
        self.ag_gemm(stream)
        return self.gemm_rs(stream)

    def reference_forward(self, x_local: torch.Tensor) -> torch.Tensor:
        """The oracle's partial on this rank, summed over the ranks by the library's reduce-scatter."""
        xg = torch.empty(self.M, self.hidden, dtype=torch.bfloat16, device=self.device)
        self.comm.all_gather(x_local.contiguous(), xg)
        part = fp8_mlp_partial_oracle(xg, self.w_gate, self.w_up, self.w2)
        out = torch.empty(self.rows, self.hidden, dtype=torch.bfloat16, device=self.device)
        self.comm.reduce_scatter(part.contiguous(), out)
        return out

    def free(self) -> None:
        torch.cuda.synchronize()
        self._x_sym.free()
        self._s_sym.free()
        self._ws.free()


class TensorParallelAttention:
    """The attention half of a tensor-parallel transformer layer with sequence-parallel activations.

    Tokens come in row-sharded ([rows_per_rank, hidden] per rank, ranks in sequence order). The column-parallel QKV
    projection runs inside the all-gather (``b200collAgGemm`` without the SwiGLU epilogue) and yields, for all
    ``n * rows_per_rank`` tokens, the ``heads / n`` query heads and ``kv_heads / n`` key/value heads this rank owns;
    rotary embedding and causal attention for those heads are local; the row-parallel output projection runs inside the
    reduce-scatter (``b200collGemmRs``) and leaves this rank's rows of the result. Together with
    :class:`TensorParallelMLP` this is a whole layer with two fused kernels per half and no stand-alone collective.
    """

    def __init__(self, comm, rows_per_rank: int, hidden: int, heads: int, kv_heads: int, seq_len: int, device=None, rope_theta: float = 500000.0,
                 std: float = 0.02, seed: int = 0, comm_ctas: int = 0):
        self.comm = comm
        self.n, self.rank = comm.nranks, comm.rank
        assert heads % self.n == 0 and kv_heads % self.n == 0, "heads and kv_heads must divide by the tensor-parallel size"
        self.rows, self.hidden, self.seq = rows_per_rank, hidden, seq_len
        self.M = self.n * rows_per_rank
        assert self.M % seq_len == 0, "the gathered tokens must be whole sequences"
        self.hq, self.hkv, self.d = heads // self.n, kv_heads // self.n, hidden // heads
        self.device = device or comm.device
        self.comm_ctas = comm_ctas
        g = torch.Generator(device=self.device).manual_seed(seed + 104729 * self.rank)
        qkv_rows = (self.hq + 2 * self.hkv) * self.d
        assert qkv_rows % 128 == 0 and (self.hq * self.d) % 64 == 0
        self.w_qkv = (torch.randn(qkv_rows, hidden, device=self.device, generator=g) * std).to(torch.bfloat16)      # q heads, k heads, v heads
        self.w_o = (torch.randn(hidden, self.hq * self.d, device=self.device, generator=g) * std).to(torch.bfloat16)
        self.rope = train_ops.rope_table(seq_len, self.d, rope_theta, self.device)
        lib = _lib_tp()
        self._x_sym = comm.sym_alloc(self.M * hidden * 2)
        self.x_full = self._x_sym.tensor((self.M, hidden), torch.bfloat16)
        self._ws = comm.sym_alloc(int(lib.b200collGemmRsWorkspaceBytes(rows_per_rank, hidden, self.n)))
        self.qkv = torch.empty(self.M, qkv_rows, dtype=torch.bfloat16, device=self.device)
        self.ctx = torch.empty(self.M, self.hq * self.d, dtype=torch.bfloat16, device=self.device)
        self.y = torch.empty(rows_per_rank, hidden, dtype=torch.bfloat16, device=self.device)
        self._dy_sym = self._ws_b = None          # backward buffers, made by the first backward()
        self._w_o_t = self._w_qkv_t = None
        self.grads: dict = {}

    def my_rows(self) -> torch.Tensor:
        return self.x_full[self.rank * self.rows:(self.rank + 1) * self.rows]

    def _attention(self, qkv: torch.Tensor) -> torch.Tensor:
        """Rotary embedding and causal attention of this rank's heads over whole sequences: qkv [M, (hq + 2 hkv) d] ->
        [M, hq d]. Differentiable (the rotary op and the attention both carry their backward)."""
        B = self.M // self.seq
        t = train_ops.rope_(qkv.view(self.M, self.hq + 2 * self.hkv, self.d), self.rope, self.hq + self.hkv)
        q = t[:, :self.hq].reshape(B, self.seq, self.hq, self.d).transpose(1, 2)
        k = t[:, self.hq:self.hq + self.hkv].reshape(B, self.seq, self.hkv, self.d).transpose(1, 2)
        v = t[:, self.hq + self.hkv:].reshape(B, self.seq, self.hkv, self.d).transpose(1, 2)
        o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.hq != self.hkv)
        return o.transpose(1, 2).reshape(self.M, self.hq * self.d)

    def _attend(self, qkv: torch.Tensor, out: torch.Tensor) -> None:
        with torch.no_grad():
            out.copy_(self._attention(qkv))

    def weights_changed(self) -> None:
        """Call after ``w_qkv`` or ``w_o`` was updated in place: the transposed copies used by ``backward`` are rebuilt."""
        self._w_o_t = self._w_qkv_t = None

    def backward(self, dy_local: torch.Tensor) -> torch.Tensor:
        """Gradients of the latest ``forward`` (its gathered input rows and its ``qkv`` must still be in place), on the
        current stream.

            d_ctx = all-gather(dy) @ w_o         one fused kernel (all-gather -> GEMM); also leaves dy of all tokens here
            d_qkv                                backward of the local rotary embedding + attention, recomputed from ``qkv``
            dx    = reduce-scatter(d_qkv @ w_qkv)   one fused kernel (GEMM -> reduce-scatter)
            dw_o  = dy^T @ ctx,  dw_qkv = d_qkv^T @ x     local GEMMs over all tokens

        Returns this rank's rows of dx; ``grads["w_qkv"]`` and ``grads["w_o"]`` hold the weight gradients."""
        lib = _lib_tp()
        s = torch.cuda.current_stream().cuda_stream
        cd = self.hq * self.d
        if self._dy_sym is None:
            assert cd % 128 == 0, "the fused kernels want this rank's head columns to be a multiple of 128"
            self._dy_sym = self.comm.sym_alloc(self.M * self.hidden * 2)
            self.dy_full = self._dy_sym.tensor((self.M, self.hidden), torch.bfloat16)
            self._ws_b = self.comm.sym_alloc(int(lib.b200collGemmRsWorkspaceBytes(self.rows, self.hidden, self.n)))
            self.dctx = torch.empty(self.M, cd, dtype=torch.bfloat16, device=self.device)
            self.dx = torch.empty(self.rows, self.hidden, dtype=torch.bfloat16, device=self.device)
        if self._w_o_t is None:
            self._w_o_t = self.w_o.t().contiguous()        # [hq d, hidden]
            self._w_qkv_t = self.w_qkv.t().contiguous()    # [hidden, (hq + 2 hkv) d]
        self.dy_full[self.rank * self.rows:(self.rank + 1) * self.rows].copy_(dy_local)
        _lib.check(lib.b200collAgGemm(self.comm.handle, self.dy_full.data_ptr(), self._w_o_t.data_ptr(), self.dctx.data_ptr(), self.rows, cd,
                                      self.hidden, 0, self.comm_ctas, s), "b200collAgGemm (backward)")
        with torch.enable_grad():
            leaf = self.qkv.detach().requires_grad_(True)
            ctx = self._attention(leaf)
            (dqkv,) = torch.autograd.grad(ctx, leaf, self.dctx)
        dqkv = dqkv.contiguous()
        _lib.check(lib.b200collGemmRs(self.comm.handle, dqkv.data_ptr(), self._w_qkv_t.data_ptr(), self._ws_b.ptr, self.dx.data_ptr(), self.rows,
                                      self.hidden, self.w_qkv.shape[0], s), "b200collGemmRs (backward)")
        train_ops.LAUNCHES += 2
        self.grads["w_o"] = train_ops.gemm(self.dy_full.t(), self.ctx.t())          # [hidden, hq d]
        self.grads["w_qkv"] = train_ops.gemm(dqkv.t(), self.x_full.t())             # [(hq + 2 hkv) d, hidden]
        return self.dx

    def forward(self, x_local: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        if x_local is not None:
            self.my_rows().copy_(x_local)
        s = (stream or torch.cuda.current_stream()).cuda_stream
        lib = _lib_tp()
        _lib.check(lib.b200collAgGemm(self.comm.handle, self.x_full.data_ptr(), self.w_qkv.data_ptr(), self.qkv.data_ptr(), self.rows, self.w_qkv.shape[0],
                                      self.hidden, 0, self.comm_ctas, s), "b200collAgGemm")
        self._attend(self.qkv, self.ctx)
        _lib.check(lib.b200collGemmRs(self.comm.handle, self.ctx.data_ptr(), self.w_o.data_ptr(), self._ws.ptr, self.y.data_ptr(), self.rows, self.hidden,
                                      self.hq * self.d, s), "b200collGemmRs")
        train_ops.LAUNCHES += 2
        return self.y

    def reference_forward(self, x_local: torch.Tensor) -> torch.Tensor:
        """Unfused: all_gather, library GEMM, the same local attention, library GEMM, reduce_scatter."""
        xg = torch.empty(self.M, self.hidden, dtype=torch.bfloat16, device=self.device)
        self.comm.all_gather(x_local.contiguous(), xg)
        qkv = xg @ self.w_qkv.t()
        ctx = torch.empty_like(self.ctx)
        self._attend(qkv, ctx)
        part = ctx @ self.w_o.t()
        out = torch.empty(self.rows, self.hidden, dtype=torch.bfloat16, device=self.device)
        self.comm.reduce_scatter(part, out)
        return out

    def free(self) -> None:
        torch.cuda.synchronize()
        self._x_sym.free()
        self._ws.free()
        if self._dy_sym is not None:
            self._dy_sym.free()
            self._ws_b.free()


class TensorParallelLayer:
    """A whole pre-norm transformer layer with tensor-parallel weights and sequence-parallel activations:

        h = x + attention(rmsnorm(x));  y = h + mlp(rmsnorm(h))

    The residual stream and both norms live on this rank's ``rows_per_rank`` tokens only; the all-gather in front of each
    half and the reduce-scatter behind it are inside the halves' GEMM kernels, in the backward pass as in the forward
    pass (four fused kernels each way and one small all-reduce per norm weight). Weights are random."""

    def __init__(self, comm, rows_per_rank: int, hidden: int, heads: int, kv_heads: int, ffn: int, seq_len: int, device=None, eps: float = 1e-5,
                 seed: int = 0, comm_ctas: int = 0):
        self.attn = TensorParallelAttention(comm, rows_per_rank, hidden, heads, kv_heads, seq_len, device, seed=seed, comm_ctas=comm_ctas)
        self.mlp = TensorParallelMLP(comm, rows_per_rank, hidden, ffn // comm.nranks, device, seed=seed + 1, comm_ctas=comm_ctas)
        dev = self.attn.device
        self.norm1 = torch.ones(hidden, dtype=torch.bfloat16, device=dev)
        self.norm2 = torch.ones(hidden, dtype=torch.bfloat16, device=dev)
        self.eps = eps
        self.comm = comm
        self.grads: dict = {}
        self._saved = None

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            h = x_local + self.attn.forward(train_ops.rmsnorm(x_local, self.norm1, self.eps))
            self._saved = (x_local, h)
            return h + self.mlp.forward(train_ops.rmsnorm(h, self.norm2, self.eps))

    def _norm_backward(self, x: torch.Tensor, w: torch.Tensor, d: torch.Tensor, name: str) -> torch.Tensor:
        with torch.enable_grad():
            xl, wl = x.detach().requires_grad_(True), w.detach().requires_grad_(True)
            dx, dw = torch.autograd.grad(train_ops.rmsnorm(xl, wl, self.eps), (xl, wl), d)
        dw = dw.float()
        if self.comm.nranks > 1:  # every rank saw its own rows only: the norm weights are replicated, their gradient is the sum
            self.comm.all_reduce(dw, op="sum")
        self.grads[name] = dw
        return dx

    def backward(self, dy_local: torch.Tensor) -> torch.Tensor:
        """Gradients of the latest ``forward``: returns this rank's rows of dx. Weight gradients land in ``attn.grads``,
        ``mlp.grads`` and (summed over the ranks, fp32) ``grads["norm1"]`` / ``grads["norm2"]``."""
        x, h = self._saved
        dh = dy_local + self._norm_backward(h, self.norm2, self.mlp.backward(dy_local), "norm2")
        return dh + self._norm_backward(x, self.norm1, self.attn.backward(dh), "norm1")

    def reference_forward(self, x_local: torch.Tensor) -> torch.Tensor:
        h = x_local + self.attn.reference_forward(train_ops.rmsnorm(x_local, self.norm1, self.eps))
        return h + self.mlp.reference_forward(train_ops.rmsnorm(h, self.norm2, self.eps))

    def free(self) -> None:
        self.attn.free()
        self.mlp.free()
