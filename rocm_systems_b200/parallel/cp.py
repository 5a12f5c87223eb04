"""Long-context building blocks on the process group: ring attention (context parallel) and the
all-to-all head/sequence re-shard (Ulysses).

The reference has neither (there is no model code in it); both are listed among the strategies a
collective stack has to carry, built from Send/Recv and AllToAll (rccl.h:731-737 grouped
send/recv, rccl.h:864-869 all-to-all). Everything here goes through ``torch.distributed``, so the
same code runs on gloo CPU ranks (tests) and on the ``b200coll`` backend (grouped Send/Recv over
NVLink FIFOs, AllToAll on the same kernel).

Both are differentiable: the communication steps are autograd functions whose backward is the
opposite transfer.

    # sequence sharded [B, H, S/P, D] on every rank
    out = ring_attention(q, k, v, group=None, causal=True)
    out = ulysses_attention(q, k, v, group=None, causal=True)
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.distributed as dist


def _exchange(send: torch.Tensor, dst: int, src: int, group) -> torch.Tensor:
    """Send ``send`` to rank ``dst`` and receive a same-shaped tensor from rank ``src`` as one grouped
    operation (both directions progress together, as grouped Send/Recv must)."""
    send = send.contiguous()
    recv = torch.empty_like(send)
    if dist.get_world_size(group) == 1:
        recv.copy_(send)
        return recv
    ops = [dist.P2POp(dist.isend, send.contiguous(), dst, group), dist.P2POp(dist.irecv, recv, src, group)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return recv


class _RingShift(torch.autograd.Function):
    """Pass a tensor to the next rank of the ring and take the previous rank's. The gradient goes
    the other way round."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        return _exchange(x, (rank + 1) % world, (rank - 1) % world, group)

    @staticmethod
    def backward(ctx, g):
        group = ctx.group
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        return _exchange(g.contiguous(), (rank - 1) % world, (rank + 1) % world, group), None


def ring_shift(x: torch.Tensor, group=None) -> torch.Tensor:
    return _RingShift.apply(x, group)


def _block_attention(q, k, v, scale: float, mask: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention of ``q`` against one key/value block in fp32: returns the un-normalised output
    ``sum_j exp(s_ij - m_i) v_j`` together with the row statistics packed as ``[m_i, l_i]``."""
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    m = s.amax(dim=-1, keepdim=True)
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))  # rows with every key masked
    p = torch.exp(s - m)
    l = p.sum(dim=-1, keepdim=True)
    return torch.matmul(p, v.float()), torch.cat([m, l], dim=-1)


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None, causal: bool = True,
                   scale: Optional[float] = None) -> torch.Tensor:
    """Blockwise attention over a sequence sharded across the ranks of ``group``.

    ``q``, ``k``, ``v`` are ``[B, H, S_local, D]`` (``k``/``v`` may have fewer heads than ``q`` for
    grouped-query attention); rank ``r`` holds tokens ``[r * S_local, (r + 1) * S_local)``. The key and
    value blocks travel once around the ring; every rank folds each visiting block into a running
    soft-max (maximum ``m``, denominator ``l``, un-normalised output), so no rank ever holds more than
    two blocks. With ``causal`` a block from a later rank contributes nothing and is skipped.
    """
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    B, H, S, D = q.shape
    if k.shape[1] != H:  # grouped-query: repeat the key/value heads
        rep = H // k.shape[1]
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    acc = torch.zeros(B, H, S, D, dtype=torch.float32, device=q.device)
    m_run = torch.full((B, H, S, 1), float("-inf"), dtype=torch.float32, device=q.device)
    l_run = torch.zeros(B, H, S, 1, dtype=torch.float32, device=q.device)
    tri = torch.ones(S, S, dtype=torch.bool, device=q.device).tril() if causal else None
    kv = torch.stack([k, v])  # one message per step
    for step in range(world):
        src = (rank - step) % world  # whose block is visiting
        if not causal or src <= rank:
            o, st = _block_attention(q, kv[0], kv[1], scale, tri if (causal and src == rank) else None)
            m_blk, l_blk = st[..., :1], st[..., 1:]
            m_new = torch.maximum(m_run, m_blk)
            a_old = torch.exp(m_run - m_new)
            a_old = torch.where(torch.isfinite(m_run), a_old, torch.zeros_like(a_old))
            a_blk = torch.exp(m_blk - m_new)
            acc = acc * a_old + o * a_blk
            l_run = l_run * a_old + l_blk * a_blk
            m_run = m_new
        elif kv.requires_grad:
            # A skipped block still has to take part in the backward ring exchange on this rank:
            # tie it into the graph with a zero weight.
            acc = acc + kv.sum() * 0.0
        if step + 1 < world:
            kv = ring_shift(kv, group)
    return (acc / l_run.clamp_min(1e-30)).to(q.dtype)


class _AllToAll(torch.autograd.Function):
    """``all_to_all_single`` over equal splits of dimension 0; the gradient is the same exchange."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.contiguous()
        out = torch.empty_like(x)
        if dist.get_world_size(group) == 1:
            return out.copy_(x)
        dist.all_to_all_single(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()  # the incoming gradient may be a permuted view; the exchange splits dimension 0 of dense memory
        out = torch.empty_like(g)
        if dist.get_world_size(ctx.group) == 1:
            return out.copy_(g), None
        dist.all_to_all_single(out, g, group=ctx.group)
        return out, None


def seq_to_heads(x: torch.Tensor, group=None) -> torch.Tensor:
    """``[B, H, S/P, D]`` (sequence sharded) -> ``[B, H/P, S, D]`` (heads sharded)."""
    P = dist.get_world_size(group)
    B, H, s, D = x.shape
    assert H % P == 0, "heads must divide by the group size"
    t = x.reshape(B, P, H // P, s, D).permute(1, 0, 2, 3, 4).contiguous()  # [P(dest), B, H/P, s, D]
    t = _AllToAll.apply(t, group)                                          # [P(source = sequence block), ...]
    return t.permute(1, 2, 0, 3, 4).reshape(B, H // P, P * s, D)


def heads_to_seq(x: torch.Tensor, group=None) -> torch.Tensor:
    """Inverse of :func:`seq_to_heads`."""
    P = dist.get_world_size(group)
    B, h, S, D = x.shape
    assert S % P == 0
    t = x.reshape(B, h, P, S // P, D).permute(2, 0, 1, 3, 4).contiguous()  # [P(dest sequence block), B, h, s, D]
    t = _AllToAll.apply(t, group)                                          # [P(source = head block), ...]
    return t.permute(1, 0, 2, 3, 4).reshape(B, P * h, S // P, D)


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None, causal: bool = True) -> torch.Tensor:
    """Attention over a sequence-sharded input by re-sharding to heads with one all-to-all per
    tensor, running ordinary attention on whole sequences, and re-sharding back."""
    qh, kh, vh = seq_to_heads(q, group), seq_to_heads(k, group), seq_to_heads(v, group)
    o = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, enable_gqa=kh.shape[1] != qh.shape[1])
    return heads_to_seq(o, group)
