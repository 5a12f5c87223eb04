"""Llama-architecture decoder trained with the FSDP engine of this package.

The model is a list of flat parameter units (embedding, one per layer, head). The forward and
backward passes are driven unit by unit so that parameter all-gathers run one unit ahead of the
compute and gradient reduce-scatters plus the optimizer run behind it, on the communication
stream (see :mod:`rocm_systems_b200.parallel.fsdp`). Every linear layer's three GEMMs (forward, input
gradient, weight gradient) run on this package's tcgen05 CTA-pair kernel, which reads row-major and
transposed operands alike, with the weight gradient written straight into the unit's flat gradient
buffer (``set_gemm("library")`` switches them to cuBLAS through ``torch.mm`` for comparison);
attention is the library SDPA kernel; norms, rotary embedding, SwiGLU, the loss, the embedding
and AdamW are this package's CUDA kernels (:mod:`rocm_systems_b200.ops.train_ops`).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F

from ..ops import train_ops as ops
from ..parallel.fsdp import AdamWConfig, FlatUnit, FSDPEngine, ParamSpec


@dataclass
class LlamaConfig:
    """Shape of a Llama-style decoder (grouped-query attention, SwiGLU MLP, RMSNorm, rotary embedding, untied output matrix)."""

    vocab: int = 128256
    hidden: int = 4096
    layers: int = 32
    heads: int = 32
    kv_heads: int = 8
    ffn: int = 14336
    rope_theta: float = 500000.0
    eps: float = 1e-5
    seq_len: int = 4096
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def llama3_70b() -> "LlamaConfig":
        return LlamaConfig(hidden=8192, layers=80, heads=64, kv_heads=8, ffn=28672, seq_len=8192)

    @staticmethod
    def llama32_1b() -> "LlamaConfig":
        return LlamaConfig(hidden=2048, layers=16, heads=32, kv_heads=8, ffn=8192, seq_len=4096)

    @staticmethod
    def llama32_3b() -> "LlamaConfig":
        return LlamaConfig(hidden=3072, layers=28, heads=24, kv_heads=8, ffn=8192, seq_len=4096)

    @staticmethod
    def llama2_7b() -> "LlamaConfig":
        return LlamaConfig(vocab=32000, hidden=4096, layers=32, heads=32, kv_heads=32, ffn=11008, rope_theta=10000.0, seq_len=4096)

    @staticmethod
    def by_name(name: str) -> "LlamaConfig":
        table = {"llama3-8b": LlamaConfig.llama3_8b, "llama3-70b": LlamaConfig.llama3_70b, "llama3.2-1b": LlamaConfig.llama32_1b,
                 "llama3.2-3b": LlamaConfig.llama32_3b, "llama2-7b": LlamaConfig.llama2_7b, "tiny": LlamaConfig.tiny}
        if name not in table:
            raise KeyError(f"unknown model {name!r}; known: {', '.join(sorted(table))}")
        return table[name]()

    def memory_per_gpu_gib(self, world: int, micro_tokens: int) -> dict:
        """A planning estimate for ZeRO-3 training on ``world`` GPUs: persistent state per GPU (bf16 shard, fp32 master
        and both AdamW moments: 14 bytes per parameter / world), the two gathered units alive at once, and the
        activations kept for backward (about 34 bytes per token, layer and hidden channel with bf16 activations and no
        recomputation, plus the logits)."""
        params = self.param_count()
        d = self.head_dim
        unit = self.hidden * (self.heads + 2 * self.kv_heads) * d + self.hidden * self.hidden + 3 * self.hidden * self.ffn + 2 * self.hidden
        unit = max(unit, self.vocab * self.hidden)
        state = 14.0 * params / world
        gathered = 2 * 2.0 * unit + 2.0 * unit          # two parameter buffers and one gradient buffer
        acts = micro_tokens * (34.0 * self.hidden * self.layers + 6.0 * self.vocab)
        gib = 1 << 30
        return {"state": state / gib, "gathered": gathered / gib, "activations": acts / gib, "total": (state + gathered + acts) / gib}

    @staticmethod
    def tiny(seq_len: int = 128) -> "LlamaConfig":
        return LlamaConfig(vocab=1024, hidden=256, layers=2, heads=4, kv_heads=2, ffn=512, seq_len=seq_len)

    def param_count(self) -> int:
        d = self.head_dim
        per_layer = self.hidden * (self.heads + 2 * self.kv_heads) * d + self.hidden * self.hidden + 3 * self.hidden * self.ffn + 2 * self.hidden
        return 2 * self.vocab * self.hidden + self.layers * per_layer + self.hidden

    def flops_per_token(self) -> float:
        """Training FLOPs per token: 6 per parameter in the GEMMs plus causal attention."""
        d = self.head_dim
        gemm_params = self.layers * (self.hidden * (self.heads + 2 * self.kv_heads) * d + self.hidden * self.hidden + 3 * self.hidden * self.ffn) + self.vocab * self.hidden
        attn = self.layers * 6 * self.seq_len * self.hidden  # 2*S*H fwd for QK^T and PV, halved by causality, x3 for fwd+bwd
        return 6.0 * gemm_params + attn


_GEMM = {"impl": os.environ.get("B200_LINEAR_GEMM", "own")}


def set_gemm(impl: str) -> None:
    """``"own"``: the linear layers run on this package's tcgen05 kernel (default); ``"library"``: on cuBLAS via ``torch.mm``."""
    assert impl in ("own", "library")
    _GEMM["impl"] = impl


def mm_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a @ b.T`` for bf16 ``a`` [M, K], ``b`` [N, K], each row-major or the transposed view of a row-major matrix."""
    if _GEMM["impl"] == "own" and a.is_cuda:
        return ops.gemm(a, b, out=out)
    return torch.mm(a, b.t(), out=out) if out is not None else torch.mm(a, b.t())


def _rm(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


class _LinearWG(torch.autograd.Function):
    """``y = x @ w.T`` whose backward writes dW into ``w.grad_view`` (a slice of the unit's flat
    gradient buffer) instead of returning a fresh tensor: no accumulate pass over the weights."""

    @staticmethod
    def forward(ctx, x, w):
        x = _rm(x)
        ctx.save_for_backward(x, w)
        return mm_nt(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy if dy.is_contiguous() else dy.contiguous()
        dx = mm_nt(dy, w.t())                       # dy [T, N] . w [N, K]
        gv = getattr(w, "grad_view", None)
        if gv is None:
            return dx, mm_nt(dy.t(), x.t())
        if getattr(w, "grad_accumulate", False):
            gv.addmm_(dy.t(), x)
        else:
            mm_nt(dy.t(), x.t(), out=gv)            # dy^T [N, T] . x [T, K]
            w.grad_accumulate = True
        return dx, None


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return _LinearWG.apply(x, w)


class _SplitQKV(torch.autograd.Function):
    """``[B, S, nh + 2 nkv, d]`` -> q, k, v as ``[B, heads, S, d]`` views. The backward writes the three
    gradients into one buffer with three strided copies; slicing through autograd would zero-fill a
    full-size tensor per slice and then add them up."""

    @staticmethod
    def forward(ctx, qkv4, nh, nkv):
        ctx.nh, ctx.nkv = nh, nkv
        return (qkv4[:, :, :nh].transpose(1, 2), qkv4[:, :, nh:nh + nkv].transpose(1, 2), qkv4[:, :, nh + nkv:].transpose(1, 2))

    @staticmethod
    def backward(ctx, dq, dk, dv):
        nh, nkv = ctx.nh, ctx.nkv
        B, _, S, d = dq.shape
        out = torch.empty(B, S, nh + 2 * nkv, d, dtype=dq.dtype, device=dq.device)
        out[:, :, :nh].copy_(dq.transpose(1, 2))
        out[:, :, nh:nh + nkv].copy_(dk.transpose(1, 2))
        out[:, :, nh + nkv:].copy_(dv.transpose(1, 2))
        return out, None, None


def layer_specs(cfg: LlamaConfig) -> List[ParamSpec]:
    d = cfg.head_dim
    return [
        ParamSpec("attn_norm", (cfg.hidden,), "ones"),
        ParamSpec("wqkv", ((cfg.heads + 2 * cfg.kv_heads) * d, cfg.hidden), std=cfg.init_std),
        ParamSpec("wo", (cfg.hidden, cfg.heads * d), std=cfg.init_std),
        ParamSpec("mlp_norm", (cfg.hidden,), "ones"),
        ParamSpec("w13", (2 * cfg.ffn, cfg.hidden), std=cfg.init_std),  # gate rows then up rows
        ParamSpec("w2", (cfg.hidden, cfg.ffn), std=cfg.init_std),
    ]


def layer_forward(p: dict, x: torch.Tensor, cfg: LlamaConfig, rope: torch.Tensor, batch: int) -> torch.Tensor:
    """One decoder layer on ``x`` [T, H] (T = batch * seq)."""
    T = x.shape[0]
    S = T // batch
    d, nh, nkv = cfg.head_dim, cfg.heads, cfg.kv_heads
    h = ops.rmsnorm(x, p["attn_norm"], cfg.eps)
    qkv = linear(h, p["wqkv"]).view(T, nh + 2 * nkv, d)
    qkv = ops.rope_(qkv, rope, nh + nkv)
    q, k, v = _SplitQKV.apply(qkv.view(batch, S, nh + 2 * nkv, d), nh, nkv)
    a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=nkv != nh)
    a = a.transpose(1, 2).reshape(T, nh * d)
    x = x + linear(a, p["wo"])
    h = ops.rmsnorm(x, p["mlp_norm"], cfg.eps)
    x = x + linear(ops.swiglu(linear(h, p["w13"])), p["w2"])
    return x


class LlamaTrainer:
    """The public training API: ``loss = trainer.step(tokens, targets)`` with host tensors in
    pinned memory or device tensors; ``loss`` is a host float when ``return_loss`` is set."""

    def __init__(self, cfg: LlamaConfig, comm=None, device: Optional[torch.device] = None, opt: Optional[AdamWConfig] = None,
                 seed: int = 0, fused_rs: bool = True, sym_shards: bool = True, overlap: bool = True, copy_engine_gather: Optional[bool] = None):
        self.cfg = cfg
        self.comm = comm
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        rank = comm.rank if comm is not None else 0
        world = comm.nranks if comm is not None else 1
        self.rank, self.world = rank, world
        with torch.cuda.device(self.device):
            units: List[FlatUnit] = []
            units.append(FlatUnit("embed", [ParamSpec("tok", (cfg.vocab, cfg.hidden), std=cfg.init_std)], rank, world, self.device, seed))
            for i in range(cfg.layers):
                units.append(FlatUnit(f"layer{i}", layer_specs(cfg), rank, world, self.device, seed + 1 + i))
            units.append(FlatUnit("head", [ParamSpec("norm", (cfg.hidden,), "ones"), ParamSpec("out", (cfg.vocab, cfg.hidden), std=cfg.init_std)],
                                  rank, world, self.device, seed + 1 + cfg.layers))
            self.engine = FSDPEngine(comm, units, opt or AdamWConfig(), fused_rs=fused_rs, sym_shards=sym_shards, overlap=overlap,
                                     copy_engine_gather=copy_engine_gather)
            self.rope = ops.rope_table(cfg.seq_len, cfg.head_dim, cfg.rope_theta, self.device)
        self.embed, self.layers, self.head = units[0], units[1:-1], units[-1]
        self._tok_dev: Optional[torch.Tensor] = None
        self._tgt_dev: Optional[torch.Tensor] = None
        self._loss_host = torch.zeros(1, dtype=torch.float32).pin_memory() if torch.cuda.is_available() else torch.zeros(1)

    # ---- one optimisation step ---------------------------------------------------------------------
    def step(self, tokens: torch.Tensor, targets: torch.Tensor, return_loss: bool = True):
        cfg, eng = self.cfg, self.engine
        with torch.cuda.device(self.device):
            if not tokens.is_cuda:
                if self._tok_dev is None or self._tok_dev.shape != tokens.shape:
                    self._tok_dev = torch.empty(tokens.shape, dtype=torch.int64, device=self.device)
                    self._tgt_dev = torch.empty(targets.shape, dtype=torch.int64, device=self.device)
                self._tok_dev.copy_(tokens, non_blocking=True)
                self._tgt_dev.copy_(targets, non_blocking=True)
                tokens, targets = self._tok_dev, self._tgt_dev
            batch, S = tokens.shape
            T = batch * S
            tok = tokens.reshape(T)
            tgt = targets.reshape(T)

            # ---- forward ----
            eng.wait_params(self.embed)
            eng.prefetch(self.layers[0])
            x = ops.embedding(tok, self.embed.params["tok"])
            if eng.reshard:
                eng.release(self.embed)
            inputs, outputs = [], []
            units = self.layers
            for i, u in enumerate(units):
                eng.wait_params(u)
                eng.prefetch(units[i + 1] if i + 1 < len(units) else self.head)
                xin = x.detach().requires_grad_(True)
                with torch.enable_grad():
                    y = layer_forward(u.params, xin, cfg, self.rope, batch)
                inputs.append(xin)
                outputs.append(y)
                x = y
                if eng.reshard and i + 1 < len(units):
                    eng.release(u)

            # ---- head: norm, logits, loss and logit gradient in place, then back through the head ----
            eng.wait_params(self.head)
            hin = x.detach().requires_grad_(True)
            with torch.enable_grad():
                hn = ops.rmsnorm(hin, self.head.params["norm"], cfg.eps)
            w_out = self.head.params["out"].detach()  # the head GEMMs are differentiated by hand below
            logits = mm_nt(hn.detach(), w_out)
            loss_rows = ops.cross_entropy_inplace(logits, tgt, 1.0 / T)
            loss = loss_rows.mean()
            eng.alloc_grad(self.head)
            dhn = mm_nt(logits, w_out.t())
            mm_nt(logits.t(), hn.detach().t(), out=self.head.grad_view("out"))
            del logits
            self.head.params["norm"].grad = None
            torch.autograd.backward(hn, dhn)
            self.head.grad_view("norm").copy_(self.head.params["norm"].grad)
            self.head.params["norm"].grad = None
            g = hin.grad
            eng.reduce_and_step(self.head)
            if eng.reshard:
                eng.release(self.head)

            # ---- backward through the layers, last to first ----
            for i in range(len(units) - 1, -1, -1):
                u = units[i]
                eng.wait_params(u)
                if i > 0:
                    eng.prefetch(units[i - 1])
                eng.alloc_grad(u)
                for name, prm in u.params.items():
                    prm.grad = None
                    if prm.dim() == 2:
                        prm.grad_view = u.grad_view(name)
                        prm.grad_accumulate = False
                torch.autograd.backward(outputs[i], g)
                for name, prm in u.params.items():
                    if prm.dim() == 1:
                        u.grad_view(name).copy_(prm.grad)
                        prm.grad = None
                    else:
                        prm.grad_view = None
                g = inputs[i].grad
                outputs[i] = None
                inputs[i] = None
                eng.reduce_and_step(u)
                if eng.reshard:
                    eng.release(u)

            # ---- embedding gradient (fp32, rows repeat) ----
            dtable = torch.zeros(self.embed.padded, dtype=torch.float32, device=self.device)
            ops.embedding_bwd_(tok, g, dtable[: cfg.vocab * cfg.hidden].view(cfg.vocab, cfg.hidden))
            eng.reduce_and_step(self.embed, fp32_full_grad=dtable)
            eng.prefetch(self.embed)  # next step starts with it
            eng.finish_step()
            if return_loss:
                self._loss_host.copy_(loss.detach().reshape(1), non_blocking=True)
                torch.cuda.current_stream().synchronize()
                return float(self._loss_host.item())
            return loss

    def eval_loss(self, tokens: torch.Tensor, targets: torch.Tensor) -> float:
        """Forward only (no update); used by tests to watch the loss go down."""
        cfg, eng = self.cfg, self.engine
        with torch.cuda.device(self.device), torch.no_grad():
            tokens, targets = tokens.to(self.device), targets.to(self.device)
            batch, S = tokens.shape
            eng.wait_params(self.embed)
            x = ops.embedding(tokens.reshape(-1), self.embed.params["tok"])
            for u in self.layers:
                eng.wait_params(u)
                x = layer_forward(u.params, x, cfg, self.rope, batch)
                if eng.reshard:
                    eng.release(u)
            eng.wait_params(self.head)
            hn = ops.rmsnorm(x, self.head.params["norm"], cfg.eps)
            logits = mm_nt(hn, self.head.params["out"])
            out = float(F.cross_entropy(logits.float(), targets.reshape(-1)).item())
            if eng.reshard:
                eng.release(self.head)
                eng.release(self.embed)
            return out

    def memory_summary(self) -> dict:
        return {"allocated_gb": torch.cuda.memory_allocated(self.device) / 2 ** 30, "peak_gb": torch.cuda.max_memory_allocated(self.device) / 2 ** 30}
