"""Fully-sharded data parallelism (ZeRO-3) over the native communicator.

Each *unit* (a transformer layer, the embedding, the head) owns one flat bf16 parameter buffer.
Every rank keeps 1/N of it (its shard) together with the fp32 master copy and both AdamW moments
of that shard. Around the compute of a unit the engine

* all-gathers the bf16 shards into the unit's full flat buffer on a communication stream, one
  unit ahead of the compute stream (prefetch), and frees the buffer afterwards;
* reduce-scatters the unit's flat bf16 gradient into an fp32 gradient shard, scaled by 1/N, on
  the communication stream while the compute stream runs the backward of the previous unit;
* applies AdamW to the shard right behind the reduce-scatter (optimizer-in-backward), which
  updates the fp32 master weights, both moments and the bf16 shard in one kernel.

With one rank the gather and the scatter disappear: the full buffer *is* the shard.
The reference has no training-side parallelism at all; this implements the FSDP/ZeRO-3 configuration
of the benchmark on the collective library in this package.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import train_ops as ops

ALIGN = 8  # elements: every parameter starts on a 16-byte boundary inside the flat buffer


@dataclass
class ParamSpec:
    """Name, shape and initialisation of one parameter inside a unit's flat buffer."""

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"  # "normal" (std below) or "ones"
    std: float = 0.02

    @property
    def numel(self) -> int:
        return int(math.prod(self.shape))


@dataclass
class AdamWConfig:
    """AdamW hyper-parameters; ``lr`` is read at every unit's update, so a schedule may change it between steps."""

    lr: float = 3e-4
    betas: Tuple[float, float] = (0.9, 0.95)
    eps: float = 1e-8
    weight_decay: float = 0.1
    max_grad_norm: Optional[float] = None  # clip the global gradient norm to this; None: every unit updates right behind its reduce-scatter


class FlatUnit:
    """One gather / reduce-scatter unit (an embedding, a layer, the head): all its parameters in one flat bf16 buffer padded
    to a multiple of the world size, of which this rank keeps a shard (bf16 for the all-gather, fp32 master copy and AdamW
    moments for the update). ``params`` are views into the full buffer, valid while it is gathered.
    """

    def __init__(self, name: str, specs: Sequence[ParamSpec], rank: int, world: int, device, seed: int):
        self.name, self.specs, self.rank, self.world, self.device = name, list(specs), rank, world, device
        offs, o = {}, 0
        for s in self.specs:
            offs[s.name] = o
            o += (s.numel + ALIGN - 1) // ALIGN * ALIGN
        self.offsets = offs
        self.numel = o
        # Ranges of the flat buffer no parameter covers (alignment gaps and the tail padding).
        self.gaps: List[Tuple[int, int]] = []
        for sp in self.specs:
            end = offs[sp.name] + sp.numel
            nxt = (end + ALIGN - 1) // ALIGN * ALIGN
            if nxt > end:
                self.gaps.append((end, nxt))
        per = (o + world - 1) // world
        self.shard_numel = (per + ALIGN - 1) // ALIGN * ALIGN
        self.padded = self.shard_numel * world
        if self.padded > o:
            self.gaps.append((o, self.padded))
        # Same full-precision initial values on every rank, then keep only this rank's slice.
        g = torch.Generator(device=device).manual_seed(seed)
        lo, hi = rank * self.shard_numel, (rank + 1) * self.shard_numel
        master = torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
        for s in self.specs:
            a, b = offs[s.name], offs[s.name] + s.numel
            if s.init == "ones":
                vals = torch.ones(s.numel, dtype=torch.float32, device=device)
            else:
                vals = torch.randn(s.numel, dtype=torch.float32, device=device, generator=g) * s.std
            i0, i1 = max(a, lo), min(b, hi)
            if i0 < i1:
                master[i0 - lo:i1 - lo] = vals[i0 - a:i1 - a]
            del vals
        self.master = master
        self.m = torch.zeros_like(master)
        self.v = torch.zeros_like(master)
        self.shard = master.to(torch.bfloat16)
        self.grad_shard: Optional[torch.Tensor] = None
        if world == 1:
            self.full = self.shard  # no gather needed
        else:
            self.full = torch.empty(self.padded, dtype=torch.bfloat16, device=device)
        self.gathered = world == 1
        self.gather_event: Optional[torch.cuda.Event] = None
        self.full_grad: Optional[torch.Tensor] = None
        # Leaf tensors viewing the full buffer; they survive storage resizes.
        self.params: Dict[str, torch.Tensor] = {}
        for s in self.specs:
            v = self.full.detach()[offs[s.name]:offs[s.name] + s.numel].view(*s.shape)
            v.requires_grad_(True)
            self.params[s.name] = v
        if world > 1:
            self.full.untyped_storage().resize_(0)  # views made above stay valid across resizes

    def grad_view(self, name: str) -> torch.Tensor:
        s = next(sp for sp in self.specs if sp.name == name)
        o = self.offsets[name]
        return self.full_grad[o:o + s.numel].view(*s.shape)

    @property
    def nbytes_full(self) -> int:
        return self.padded * 2


class FSDPEngine:
    """Owns the units, the communication stream and the schedule primitives."""

    def __init__(self, comm, units: List[FlatUnit], opt: AdamWConfig, reshard_after_forward: bool = True, fused_rs: bool = True,
                 sym_shards: bool = True, overlap: bool = True, copy_engine_gather: Optional[bool] = None):
        self.comm, self.units, self.opt = comm, units, opt
        self.world = comm.nranks if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        self.reshard = reshard_after_forward and self.world > 1
        # overlap=False runs gathers, reductions and updates on the compute stream itself: the schedule of a step becomes
        # strictly sequential, which is what a result obtained with overlap is checked against.
        self.comm_stream = torch.cuda.Stream(priority=-1) if overlap else torch.cuda.current_stream()
        self.step_count = 0
        self.fused_rs = fused_rs
        self._pending: List[torch.cuda.Event] = []
        self._sym_shards = None
        self._grad_slots = None
        # Global-norm clipping: the update of every unit waits for the norm of all of them.
        self._held: List[tuple] = []          # (unit, reduced gradient shard) until finish_step
        self._sumsq: Optional[torch.Tensor] = None
        self.last_grad_norm: Optional[torch.Tensor] = None   # device scalar of the latest step (before clipping)
        # With the shards in symmetric memory the parameter all-gather can be made by the copy engines: one peer-to-peer
        # copy per peer behind a tiny barrier kernel, so that no SM is taken from the GEMMs it overlaps (8B model on 2 GPUs:
        # 212 ms per step against 224 ms with the all-gather kernel, and 215 ms on one GPU). That is the default between
        # two ranks. On four GPUs the one run of this mode ended in a bounded-wait report (lanes of the reduce-scatter
        # kernel of one rank not arriving within 5 s; the cause is not understood), so from three
        # ranks up the default stays the all-gather kernel; copy_engine_gather=True forces the copies.
        self.copy_engine_gather = False
        if sym_shards and self.world > 1 and hasattr(comm, "sym_alloc"):
            self._place_shards_in_symmetric_memory()
            self.copy_engine_gather = (self.world == 2) if copy_engine_gather is None else bool(copy_engine_gather)

    def _place_shards_in_symmetric_memory(self) -> None:
        """Move every unit's bf16 shard into one symmetric allocation. The parameter all-gather then
        reads the peers' shards in place (the zero-copy path of the collective engine) instead of
        staging them; AdamW keeps writing the shard where it now lives. The default on two or more
        ranks (measured on 2 GPUs with the 8B model: 227 ms per step against 252 ms staged); it changes
        where 16 GB / N of memory comes from, not what is computed."""
        align = 256
        offs, total = [], 0
        for u in self.units:
            offs.append(total)
            total += (u.shard_numel * 2 + align - 1) // align * align
        self._sym_shards = self.comm.sym_alloc(total)
        for u, o in zip(self.units, offs):
            t = self._sym_shards.tensor((u.shard_numel,), torch.bfloat16, offset_bytes=o)
            t.copy_(u.shard)
            u.shard = t
            u.peer_shards = [self._sym_shards.tensor((u.shard_numel,), torch.bfloat16, offset_bytes=o, peer=p) for p in range(self.world)]
        # Two symmetric gradient buffers, used alternately by consecutive units: the fused
        # reduce-scatter then reads the peers' gradients in place. A buffer is handed out again only
        # after the reduce-scatter that read it has finished (its kernel ends with a barrier, so by
        # then no peer reads this rank's copy either).
        slot_elems = max(u.padded for u in self.units)
        slot_bytes = (slot_elems * 2 + align - 1) // align * align
        self._sym_grads = self.comm.sym_alloc(2 * slot_bytes)
        self._grad_slots = [self._sym_grads.tensor((slot_elems,), torch.bfloat16, offset_bytes=i * slot_bytes) for i in range(2)]
        self._grad_slot_done = [None, None]
        self._grad_slot_next = 0
        torch.cuda.synchronize()
        self.comm.host_barrier()  # every rank's shards are in place before anyone gathers

    # ---- parameters -----------------------------------------------------------------------------
    def prefetch(self, unit: FlatUnit) -> None:
        """Start the all-gather of ``unit`` on the communication stream (no-op when gathered)."""
        if unit.gathered:
            return
        unit.full.untyped_storage().resize_(unit.nbytes_full)
        self.comm_stream.wait_stream(torch.cuda.current_stream())  # the memory may be recycled compute memory
        with torch.cuda.stream(self.comm_stream):
            if self.copy_engine_gather:
                # Every rank's shard is final once its communication stream reaches this barrier (its AdamW of this unit
                # ran earlier on that stream). A shard is next written behind the unit's gradient reduce-scatter, a
                # collective that no rank enters before it has used the gathered parameters, so no closing barrier is needed.
                self.comm.barrier(stream=self.comm_stream)
                n = unit.shard_numel
                # a second tensor over the same memory: like the collective kernels, the copies must not count as in-place
                # modifications of the parameter views that a saved forward pass still refers to
                from ..comm import _tensor_from_ptr

                dst = _tensor_from_ptr(unit.full.data_ptr(), (self.world * n,), torch.bfloat16, unit.device)
                for i in range(self.world):
                    p = (self.rank + i) % self.world
                    dst[p * n:(p + 1) * n].copy_(unit.peer_shards[p], non_blocking=True)
            else:
                self.comm.all_gather(unit.shard, unit.full, stream=self.comm_stream)
            ev = torch.cuda.Event()
            ev.record(self.comm_stream)
        unit.gather_event = ev
        unit.gathered = True

    def wait_params(self, unit: FlatUnit) -> None:
        """Make the compute stream wait until ``unit``'s parameters are in place."""
        if not unit.gathered:
            self.prefetch(unit)
        if unit.gather_event is not None:
            torch.cuda.current_stream().wait_event(unit.gather_event)
            unit.gather_event = None

    def release(self, unit: FlatUnit) -> None:
        """Free the full parameter buffer (the shard stays)."""
        if self.world == 1 or not unit.gathered:
            return
        unit.full.untyped_storage().resize_(0)
        unit.gathered = False

    # ---- gradients --------------------------------------------------------------------------------
    def alloc_grad(self, unit: FlatUnit) -> None:
        """The flat gradient buffer of ``unit``. Every parameter's gradient is written (not
        accumulated) into its view by the backward pass, so only the gaps need zeroing."""
        if self._grad_slots is not None:
            slot = self._grad_slot_next
            self._grad_slot_next ^= 1
            if self._grad_slot_done[slot] is not None:
                torch.cuda.current_stream().wait_event(self._grad_slot_done[slot])
            unit.full_grad = self._grad_slots[slot][:unit.padded]
            unit.grad_slot = slot
        else:
            unit.full_grad = torch.empty(unit.padded, dtype=torch.bfloat16, device=unit.device)
            unit.grad_slot = None
        for a, b in unit.gaps:
            unit.full_grad[a:b].zero_()

    def reduce_and_step(self, unit: FlatUnit, fp32_full_grad: Optional[torch.Tensor] = None) -> None:
        """Reduce-scatter ``unit``'s gradient (mean over ranks) into fp32 and apply AdamW to the
        shard, all on the communication stream behind the compute already queued."""
        o = self.opt
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.comm_stream.wait_event(ev)
        src = fp32_full_grad if fp32_full_grad is not None else unit.full_grad
        with torch.cuda.stream(self.comm_stream):
            gshard = None
            if self.world > 1:
                gshard = torch.empty(unit.shard_numel, dtype=torch.float32, device=unit.device)
            if fp32_full_grad is not None:
                if self.world == 1:
                    gshard = fp32_full_grad[:unit.shard_numel]
                else:
                    self.comm.reduce_scatter(fp32_full_grad, gshard, op="avg", stream=self.comm_stream)
            elif self.world == 1:
                gshard = unit.full_grad[:unit.shard_numel]  # AdamW reads the bf16 gradient directly
            elif self.fused_rs:
                from ..ops import comm_ops

                comm_ops.reduce_scatter_cast(self.comm, unit.full_grad, gshard, 1.0 / self.world, stream=self.comm_stream)
            else:
                tmp = torch.empty(unit.shard_numel, dtype=torch.bfloat16, device=unit.device)
                self.comm.reduce_scatter(unit.full_grad, tmp, op="avg", stream=self.comm_stream)
                ops.cast_scale_(tmp, gshard, 1.0)
            if fp32_full_grad is None and getattr(unit, "grad_slot", None) is not None:
                read = torch.cuda.Event()
                read.record(self.comm_stream)  # the reduce-scatter is behind us on this stream: the buffer may be reused after it
                self._grad_slot_done[unit.grad_slot] = read
            if o.max_grad_norm is not None:
                sq = torch.sum(gshard.float() ** 2) if gshard.dtype != torch.float32 else torch.dot(gshard, gshard)
                self._sumsq = sq if self._sumsq is None else self._sumsq + sq
                self._held.append((unit, gshard))
            else:
                ops.adamw_(unit.master, unit.m, unit.v, gshard, unit.shard, o.lr, o.betas, o.eps, o.weight_decay, self.step_count + 1)
            done = torch.cuda.Event()
            done.record(self.comm_stream)
        src.record_stream(self.comm_stream)
        unit.full_grad = None
        self._pending.append(done)

    def _clip_and_update(self) -> None:
        """With ``max_grad_norm``: sum the squared norms over the ranks, scale every held gradient shard by
        ``min(1, max_norm / norm)`` on the device (no host round trip) and run the deferred AdamW updates."""
        o = self.opt
        with torch.cuda.stream(self.comm_stream):
            total = self._sumsq.reshape(1).float()
            if self.world > 1:
                self.comm.all_reduce(total, op="sum", stream=self.comm_stream)
            norm = total.sqrt()
            coef = (o.max_grad_norm / (norm + 1e-6)).clamp(max=1.0)
            self.last_grad_norm = norm
            for unit, gshard in self._held:
                gshard.mul_(coef.to(gshard.dtype))
                ops.adamw_(unit.master, unit.m, unit.v, gshard, unit.shard, o.lr, o.betas, o.eps, o.weight_decay, self.step_count + 1)
            done = torch.cuda.Event()
            done.record(self.comm_stream)
        self._held.clear()
        self._sumsq = None
        self._pending.append(done)

    def finish_step(self) -> None:
        """Join the communication stream: after this the shards hold the updated weights."""
        if self._held:
            self._clip_and_update()
        cur = torch.cuda.current_stream()
        for ev in self._pending:
            cur.wait_event(ev)
        self._pending.clear()
        self.step_count += 1

    # ---- checkpoint ---------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"step": self.step_count, "world": self.world, "rank": self.rank,
                "units": {u.name: {"master": u.master.cpu(), "m": u.m.cpu(), "v": u.v.cpu()} for u in self.units}}

    def load_state_dict(self, sd: dict) -> None:
        assert sd["world"] == self.world and sd["rank"] == self.rank, "sharded checkpoint belongs to another layout"
        self.step_count = sd["step"]
        for u in self.units:
            s = sd["units"][u.name]
            u.master.copy_(s["master"])
            u.m.copy_(s["m"])
            u.v.copy_(s["v"])
            u.shard.copy_(u.master.to(torch.bfloat16))
