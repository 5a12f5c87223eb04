"""Expert-parallel mixture-of-experts layer on the fused dispatch / combine kernels.

``MoELayer`` owns this rank's experts (``experts_local`` of ``nranks * experts_local``) and one
symmetric window. ``forward(x, router_logits)`` runs route -> dispatch (fp8 e4m3, one scale per
128 channels, device-initiated puts) -> grouped expert GEMMs on tcgen05 with SwiGLU -> combine
(pull + gate-weighted sum in bf16 output) on the current stream. ``reference_forward`` is the
same computation in plain PyTorch (all_to_all of this package for the exchange) and serves as
oracle and timing baseline.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ..ops import train_ops
from .tp import deinterleave_gate_up, interleave_gate_up

_done = False


def _lib_ep():
    global _done
    lib = _lib.load()
    if not _done:
        vp, i32 = ctypes.c_void_p, ctypes.c_int
        lib.b200collEpWorkspaceBytes.argtypes = [i32] * 5
        lib.b200collEpWorkspaceBytes.restype = ctypes.c_size_t
        lib.b200collEpRoute.argtypes = [vp, vp, vp, i32, i32, i32, vp]
        lib.b200collEpDispatch.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]
        lib.b200collEpExperts.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]
        lib.b200collEpExpertsFp8.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]
        lib.b200collEpCombine.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]
        lib.b200collEpCounts.argtypes = [vp, vp, i32, i32, i32, i32, vp, vp, vp]
        lib.b200collEpGateGrad.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]
        lib.b200collEpGatherGrad.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]
        lib.b200collEpGroupedGemm.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]
        _done = True
    return lib


def quantize_e4m3_per128(x: torch.Tensor):
    """Reference quantiser: fp8 e4m3 values and one fp32 scale per 128 channels (amax * fp32(1 / 448))."""
    T, H = x.shape
    g = x.float().view(T, H // 128, 128)
    scale = g.abs().amax(-1).clamp_min(1e-10) * (1.0 / 448.0)
    q = (g / scale.unsqueeze(-1)).to(torch.float8_e4m3fn)
    return q.view(T, H), scale


def dequantize_e4m3_per128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    T, H = q.shape
    return (q.float().view(T, H // 128, 128) * scale.unsqueeze(-1)).view(T, H).to(torch.bfloat16)


def ref_route(logits: torch.Tensor, k: int):
    """The routing rule of ``b200collEpRoute`` in plain PyTorch (any device): top ``k`` of each row, largest first, ties to
    the lower expert id; a NaN counts as -inf and +inf as the largest finite value; when fewer than ``k`` values are above
    -inf the row fills up with the lowest ids not yet taken; gate weights are the softmax over the selected values, or 1/k
    each when all of them are -inf. Every id is in [0, E) and every weight finite, whatever the row holds."""
    x = torch.nan_to_num(logits.float(), nan=float("-inf"), posinf=torch.finfo(torch.float32).max, neginf=float("-inf"))
    T, E = x.shape
    # stable descending sort = largest first, equal values in ascending id order (also among the -inf entries)
    order = torch.sort(x, dim=-1, descending=True, stable=True).indices[:, :k]
    sel = torch.gather(x, 1, order)
    flat = torch.isinf(sel[:, :1]) & (sel[:, :1] < 0)
    w = torch.softmax(torch.where(flat, torch.zeros_like(sel), sel), dim=-1)
    return order.to(torch.int32), w


def router_backward(top_w: torch.Tensor, top_idx: torch.Tensor, d_gate: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Gradient with respect to the router logits [T, E] given the gradient with respect to the gate weights [T, k]: the gate
    weights are the softmax over the k selected logits, so d_sel = w * (d_gate - sum(d_gate * w)) lands on the selected
    columns and every other column gets zero (the selection itself is piecewise constant)."""
    d_sel = top_w * (d_gate - (d_gate * top_w).sum(-1, keepdim=True))
    return torch.zeros(top_w.shape[0], num_experts, dtype=torch.float32, device=top_w.device).scatter_(1, top_idx.long(), d_sel.float())


def route(logits: torch.Tensor, k: int):
    """``b200collEpRoute`` alone: expert ids [T, k] (int32) and gate weights [T, k] (fp32) of fp32 logits [T, E] on the GPU."""
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    T, E = logits.shape
    idx = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    s = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib_ep().b200collEpRoute(logits.data_ptr(), idx.data_ptr(), w.data_ptr(), T, E, k, s), "b200collEpRoute")
    train_ops.LAUNCHES += 1
    return idx, w


class MoELayer:
    """A mixture-of-experts layer with the experts spread over the ranks of ``comm``: top-k routing, one dispatch kernel that
    permutes, quantises to fp8 e4m3 (a scale per 128 channels) and stores rows into the owning ranks, grouped expert GEMMs on
    the tcgen05 kernel, and one combine kernel that pulls the expert outputs back and applies the gate weights in a fixed
    order. ``reference_forward`` states the same layer in plain PyTorch with NCCL-style collectives.

    ``fp8_experts=True`` quantises the gate/up weights once per 128 x 128 block and runs the first expert GEMM directly on
    the fp8 rows that arrived (``b200collEpExpertsFp8``): no dequantisation pass, no bf16 copy of the received activations.

    ``backward(dy)`` (bf16 experts) returns the gradients with respect to the tokens and the router logits and leaves the
    expert weights' gradients in ``grads``. It reuses the rows and slots of the forward dispatch: the gradient of combine is
    a gather of ``gate * dy`` at the experts' ranks, the gradient of dispatch is a combine with unit weights, and the
    experts' input-gradient GEMMs are grouped GEMMs on transposed weights. The fp8 transport of the forward pass is treated
    as the identity (straight-through).
    """

    def __init__(self, comm, experts_local: int, hidden: int, ffn: int, top_k: int, tokens: int, capacity: int = 0, std: float = 0.02, seed: int = 0,
                 fp8_experts: bool = False):
        self.comm, self.n, self.rank = comm, comm.nranks, comm.rank
        self.el, self.hidden, self.ffn, self.k, self.T = experts_local, hidden, ffn, top_k, tokens
        self.E = self.n * experts_local
        dev = comm.device
        self.device = dev
        avg = max(1, self.n * tokens * top_k // self.E)
        cap = capacity or 4 * avg
        self.cap = (cap + 127) // 128 * 128
        g = torch.Generator(device=dev).manual_seed(seed + 104729 * self.rank)
        self.w_gate = (torch.randn(experts_local, ffn, hidden, device=dev, generator=g) * std).to(torch.bfloat16)
        self.w_up = (torch.randn(experts_local, ffn, hidden, device=dev, generator=g) * std).to(torch.bfloat16)
        self.w_down = (torch.randn(experts_local, hidden, ffn, device=dev, generator=g) * std).to(torch.bfloat16)
        tile = 256 if (2 * ffn) % 256 == 0 else 128
        self.w13 = torch.cat([interleave_gate_up(self.w_gate[e], self.w_up[e], tile) for e in range(experts_local)]).contiguous()
        self.w2 = self.w_down.reshape(experts_local * hidden, ffn).contiguous()
        self.fp8_experts = fp8_experts
        if fp8_experts:
            from ..ops import fp8
            w13_128 = torch.cat([interleave_gate_up(self.w_gate[e], self.w_up[e], 128) for e in range(experts_local)]).contiguous()
            self.w13_q, self.w13_s = fp8.quantize_weight(w13_128)
            # what the experts multiply by, for the oracle: the block-quantised weights back in bf16, de-interleaved
            deq = fp8.ref_dequantize_weight(self.w13_q, self.w13_s).view(experts_local, 2 * ffn // 128, 2, 64, hidden)
            self._w_gate_ref = deq[:, :, 0].reshape(experts_local, ffn, hidden).to(torch.bfloat16)
            self._w_up_ref = deq[:, :, 1].reshape(experts_local, ffn, hidden).to(torch.bfloat16)
        lib = _lib_ep()
        self._win = comm.sym_alloc(int(lib.b200collEpWorkspaceBytes(self.n, experts_local, self.cap, hidden, ffn)))
        rows = experts_local * self.cap
        self.xb = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=dev)
        self.act = torch.zeros(rows, ffn, dtype=torch.bfloat16, device=dev)
        self.top_idx = torch.empty(tokens, top_k, dtype=torch.int32, device=dev)
        self.top_w = torch.empty(tokens, top_k, dtype=torch.float32, device=dev)
        self.sent = torch.empty(tokens, top_k, dtype=torch.int32, device=dev)
        self.out = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
        self.tile = tile
        self._dy_sym = None      # backward buffers, made by the first backward()
        self._w2_t = self._w13_t = None
        self.grads: dict = {}

    def _args(self):
        return (self.el, self.cap, self.hidden, self.ffn)

    def route(self, logits: torch.Tensor) -> None:
        assert logits.dtype == torch.float32 and logits.shape == (self.T, self.E) and logits.is_contiguous()
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib_ep().b200collEpRoute(logits.data_ptr(), self.top_idx.data_ptr(), self.top_w.data_ptr(), self.T, self.E, self.k, s), "b200collEpRoute")
        train_ops.LAUNCHES += 1

    def dispatch(self, x: torch.Tensor) -> None:
        assert x.dtype == torch.bfloat16 and x.shape == (self.T, self.hidden) and x.is_contiguous()
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib_ep().b200collEpDispatch(self.comm.handle, self._win.ptr, x.data_ptr(), self.top_idx.data_ptr(), self.sent.data_ptr(), self.T,
                                                self.k, *self._args(), s), "b200collEpDispatch")
        train_ops.LAUNCHES += 1

    def experts(self) -> None:
        s = torch.cuda.current_stream().cuda_stream
        if self.fp8_experts:
            _lib.check(_lib_ep().b200collEpExpertsFp8(self.comm.handle, self._win.ptr, self.w13_q.data_ptr(), self.w13_s.data_ptr(), self.w2.data_ptr(),
                                                      self.act.data_ptr(), *self._args(), s), "b200collEpExpertsFp8")
            train_ops.LAUNCHES += 2
            return
        _lib.check(_lib_ep().b200collEpExperts(self.comm.handle, self._win.ptr, self.w13.data_ptr(), self.w2.data_ptr(), self.xb.data_ptr(),
                                               self.act.data_ptr(), *self._args(), s), "b200collEpExperts")
        train_ops.LAUNCHES += 3

    def combine(self) -> torch.Tensor:
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib_ep().b200collEpCombine(self.comm.handle, self._win.ptr, self.top_idx.data_ptr(), self.top_w.data_ptr(), self.sent.data_ptr(),
                                               self.out.data_ptr(), self.T, self.k, *self._args(), s), "b200collEpCombine")
        train_ops.LAUNCHES += 2
        return self.out

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        self.route(logits)
        self.dispatch(x)
        self.experts()
        return self.combine()

    def counts(self):
        c = (ctypes.c_uint * self.el)()
        d = ctypes.c_int()
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib_ep().b200collEpCounts(self.comm.handle, self._win.ptr, *self._args(), c, ctypes.byref(d), s), "b200collEpCounts")
        return list(c), d.value

    # ---- backward ------------------------------------------------------------------------------------------
    def weights_changed(self) -> None:
        """Call after ``w13`` or ``w2`` was updated in place: the transposed copies used by ``backward`` are rebuilt."""
        self._w2_t = self._w13_t = None

    def _grouped(self, a: torch.Tensor, w: torch.Tensor, out, w_rows: int, K: int) -> None:
        s = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib_ep().b200collEpGroupedGemm(self.comm.handle, self._win.ptr, a.data_ptr(), w.data_ptr(), out.data_ptr() if out is not None else None,
                                                   w_rows, K, *self._args(), s), "b200collEpGroupedGemm")
        train_ops.LAUNCHES += 1

    def backward(self, dy: torch.Tensor):
        """Gradients of the latest ``forward`` (bf16 experts), on the current stream: returns ``(dx [T, hidden] bf16,
        d_logits [T, E] fp32)``; ``grads["w13"]`` ([experts_local * 2 ffn, hidden], interleaved like ``w13``) and
        ``grads["w2"]`` ([experts_local * hidden, ffn]) hold the expert weights' gradients.

        One host read per call: the number of rows each local expert received (the reduction length of its two
        weight-gradient GEMMs); everything else is queued without a round trip."""
        assert not self.fp8_experts, "backward is built for the bf16 expert GEMMs (the fp8 form keeps no bf16 copy of the received rows)"
        assert dy.dtype == torch.bfloat16 and dy.shape == (self.T, self.hidden)
        lib = _lib_ep()
        s = torch.cuda.current_stream().cuda_stream
        el, cap, H, f, T, k = self.el, self.cap, self.hidden, self.ffn, self.T, self.k
        rows = el * cap
        dev = self.device
        if self._dy_sym is None:
            self._dy_sym = self.comm.sym_alloc(T * H * 2)
            self._gate_sym = self.comm.sym_alloc(T * k * 4)
            self.dy_s = self._dy_sym.tensor((T, H), torch.bfloat16)
            self.gate_s = self._gate_sym.tensor((T, k), torch.float32)
            self.d_out = torch.zeros(rows, H, dtype=torch.bfloat16, device=dev)
            self.d_act = torch.zeros(rows, f, dtype=torch.bfloat16, device=dev)
            self.gu = torch.zeros(rows, 2 * f, dtype=torch.bfloat16, device=dev)
            self.d_gate = torch.empty(T, k, dtype=torch.float32, device=dev)
            self.ones = torch.ones(T, k, dtype=torch.float32, device=dev)
            self.dx = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        if self._w2_t is None:
            self._w2_t = self.w2.view(el, H, f).transpose(1, 2).reshape(el * f, H).contiguous()          # per expert [ffn, hidden]
            self._w13_t = self.w13.view(el, 2 * f, H).transpose(1, 2).reshape(el * H, 2 * f).contiguous()  # per expert [hidden, 2 ffn]
        self.dy_s.copy_(dy)
        self.gate_s.copy_(self.top_w)
        # d gate, from the forward pass's expert outputs (still in the window's output region)
        _lib.check(lib.b200collEpGateGrad(self.comm.handle, self._win.ptr, self.dy_s.data_ptr(), self.top_idx.data_ptr(), self.sent.data_ptr(),
                                          self.d_gate.data_ptr(), T, k, *self._args(), s), "b200collEpGateGrad")
        # gradient of combine: gate * dy of every arrived row, pulled to the expert's rank
        _lib.check(lib.b200collEpGatherGrad(self.comm.handle, self._win.ptr, self._dy_sym.ptr, self._gate_sym.ptr, self.d_out.data_ptr(), T, k,
                                            *self._args(), s), "b200collEpGatherGrad")
        train_ops.LAUNCHES += 3
        self._grouped(self.d_out, self._w2_t, self.d_act, f, H)            # d_act = d_out @ w2
        self._grouped(self.xb, self.w13, self.gu, 2 * f, H)                # gate/up pre-activations again (forward kept act only)
        nt = 2 * f // self.tile
        dgu = train_ops.swiglu_bwd(self.gu.view(rows * nt, self.tile), self.d_act.view(rows * nt, self.tile // 2)).view(rows, 2 * f)
        self._grouped(dgu, self._w13_t, None, H, 2 * f)                    # d(rows) = d_gu @ w13, into the window's output region
        counts, _ = self.counts()
        dw13 = torch.zeros(el * 2 * f, H, dtype=torch.bfloat16, device=dev)
        dw2 = torch.zeros(el * H, f, dtype=torch.bfloat16, device=dev)
        for e in range(el):
            c = min(int(counts[e]), cap)
            if c == 0:
                continue
            r0 = e * cap
            train_ops.gemm(self.d_out[r0:r0 + c].t(), self.act[r0:r0 + c].t(), out=dw2[e * H:(e + 1) * H])
            train_ops.gemm(dgu[r0:r0 + c].t(), self.xb[r0:r0 + c].t(), out=dw13[e * 2 * f:(e + 1) * 2 * f])
        self.grads["w13"], self.grads["w2"] = dw13, dw2
        # gradient of dispatch: every token sums the rows of its k experts (a combine with unit weights)
        _lib.check(lib.b200collEpCombine(self.comm.handle, self._win.ptr, self.top_idx.data_ptr(), self.ones.data_ptr(), self.sent.data_ptr(),
                                         self.dx.data_ptr(), T, k, *self._args(), s), "b200collEpCombine (backward)")
        train_ops.LAUNCHES += 2
        return self.dx, router_backward(self.top_w, self.top_idx, self.d_gate, self.E)

    def expert_weight_grads(self):
        """``grads`` as (d w_gate, d w_up [experts_local, ffn, hidden], d w_down [experts_local, hidden, ffn])."""
        el, f, H = self.el, self.ffn, self.hidden
        parts = [deinterleave_gate_up(self.grads["w13"][e * 2 * f:(e + 1) * 2 * f], self.tile) for e in range(el)]
        return (torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]), self.grads["w2"].view(el, H, f))

    # ---- plain PyTorch oracle ---------------------------------------------------------------------------
    def reference_forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        n, el, k, T, H = self.n, self.el, self.k, self.T, self.hidden
        top_v, top_i = torch.topk(logits, k, dim=-1)
        w = torch.softmax(top_v, dim=-1)
        q, sc = quantize_e4m3_per128(x)
        xd = dequantize_e4m3_per128(q, sc)                      # what the experts see after fp8 transport
        flat_e = top_i.reshape(-1)                               # [T*k]
        flat_t = torch.arange(T, device=x.device).repeat_interleave(k)
        dst = flat_e // el
        order = torch.argsort(dst, stable=True)
        send_rows = xd[flat_t[order]].contiguous()
        send_e = (flat_e[order] % el).to(torch.int32).contiguous()
        send_counts = torch.bincount(dst, minlength=n).to(torch.int64)
        recv_counts = torch.empty_like(send_counts)
        self.comm.all_to_all(send_counts, recv_counts)
        sc_l, rc_l = send_counts.tolist(), recv_counts.tolist()
        sd = [sum(sc_l[:i]) for i in range(n)]
        rd = [sum(rc_l[:i]) for i in range(n)]
        R = sum(rc_l)
        recv_rows = torch.empty(max(R, 1), H, dtype=torch.bfloat16, device=x.device)
        recv_e = torch.empty(max(R, 1), dtype=torch.int32, device=x.device)
        self.comm.all_to_allv(send_rows, [c * H for c in sc_l], [d * H for d in sd], recv_rows, [c * H for c in rc_l], [d * H for d in rd])
        self.comm.all_to_allv(send_e, sc_l, sd, recv_e, rc_l, rd)
        y = torch.zeros(max(R, 1), H, dtype=torch.bfloat16, device=x.device)
        for e in range(el):
            m = (recv_e[:R] == e).nonzero().flatten()
            if m.numel() == 0:
                continue
            xe = recv_rows[m]
            wg, wu = (self._w_gate_ref[e], self._w_up_ref[e]) if self.fp8_experts else (self.w_gate[e], self.w_up[e])
            a = (torch.nn.functional.silu((xe @ wg.t()).float()) * (xe @ wu.t()).float()).to(torch.bfloat16)
            y[m] = a @ self.w_down[e].t()
        back = torch.empty(T * k, H, dtype=torch.bfloat16, device=x.device)
        self.comm.all_to_allv(y, [c * H for c in rc_l], [d * H for d in rd], back, [c * H for c in sc_l], [d * H for d in sd])
        contrib = torch.empty(T * k, H, dtype=torch.float32, device=x.device)
        contrib[order] = back.float()
        out = (contrib.view(T, k, H) * w.unsqueeze(-1)).sum(1)
        return out.to(torch.bfloat16)

    def free(self) -> None:
        torch.cuda.synchronize()
        self._win.free()
        if self._dy_sym is not None:
            self._dy_sym.free()
            self._gate_sym.free()
