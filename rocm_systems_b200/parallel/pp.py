"""Pipeline parallelism: one stage per rank, activations forward and gradients backward over
Send/Recv, micro-batches scheduled GPipe-style or 1F1B.

The reference has no pipeline code; what it defines is the transport contract this module sits on:
point-to-point operations progress concurrently only inside one group (rccl.h:731-737), which is
why every exchange here is a ``batch_isend_irecv``. On CPU ranks that is gloo; on GPUs it is this
package's ``b200coll`` backend, or stock NCCL when the caller passes a group created with
``backend="nccl"`` (stage-to-stage copies are plain bulk transfers, there is nothing to fuse).

    stage = PipelineStage(module, rank, world, group)
    losses = stage.run(micro_batches, targets, loss_fn, schedule="1f1b")   # on every rank
    optimizer.step()
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


def _batch(sends, recvs, group) -> None:
    """One grouped exchange: ``sends`` = [(tensor, dst)], ``recvs`` = [(tensor, src)]."""
    ops = [dist.P2POp(dist.isend, t, d, group) for t, d in sends] + [dist.P2POp(dist.irecv, t, r, group) for t, r in recvs]
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()


def schedule_1f1b(stage: int, stages: int, micro: int) -> List[tuple]:
    """The 1F1B order of one stage as a list of ``("F", i)`` / ``("B", i)``: ``stages - stage - 1``
    warm-up forwards, then one forward and one backward alternately, then the remaining backwards.
    At most ``stages - stage`` activations are alive at once (GPipe keeps all ``micro``)."""
    warm = min(stages - stage - 1, micro)
    order: List[tuple] = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < micro:
        order.append(("F", f))
        f += 1
        order.append(("B", b))
        b += 1
    while b < micro:
        order.append(("B", b))
        b += 1
    return order


def schedule_gpipe(stage: int, stages: int, micro: int) -> List[tuple]:
    return [("F", i) for i in range(micro)] + [("B", i) for i in range(micro)]


class PipelineStage:
    """Runs ``module`` as stage ``rank`` of a ``world``-stage pipeline.

    The first stage consumes the micro-batches, the last computes the loss; the others receive
    their input from the previous rank, whose per-micro-batch shape is ``act_shape``. In the steady
    state of 1F1B an activation going forward and the gradient coming back travel as one grouped
    exchange, so neither side can block the other. Gradients accumulate in ``module``'s parameters over the micro-batches, scaled by 1/micro.
    """

    def __init__(self, module: Callable[[torch.Tensor], torch.Tensor], rank: Optional[int] = None, world: Optional[int] = None, group=None,
                 act_shape: Optional[Sequence[int]] = None, act_dtype: torch.dtype = torch.float32, device: Optional[torch.device] = None):
        self.module, self.group = module, group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.world = dist.get_world_size(group) if world is None else world
        self.first, self.last = self.rank == 0, self.rank == self.world - 1
        self.act_shape = tuple(act_shape) if act_shape is not None else None
        self.act_dtype = act_dtype
        self.device = device or torch.device("cpu")
        self.peak_alive = 0  # most activations held at once in the last run (what 1F1B bounds)

    def run(self, micro_batches: Optional[Sequence[torch.Tensor]], targets: Optional[Sequence[torch.Tensor]],
            loss_fn: Optional[Callable[[torch.Tensor, torch.Tensor], torch.Tensor]], n_micro: Optional[int] = None,
            schedule: str = "1f1b") -> List[float]:
        """One optimizer step's worth of micro-batches. Returns the micro-batch losses on the last
        stage (empty elsewhere)."""
        micro = n_micro if n_micro is not None else len(micro_batches)
        order = (schedule_1f1b if schedule == "1f1b" else schedule_gpipe)(self.rank, self.world, micro)
        if not self.first and self.act_shape is None:
            raise ValueError("act_shape (the per-micro-batch input shape of this stage) is required on every stage but the first")
        inputs: dict = {}
        outputs: dict = {}
        acts_in: dict = {}   # activations already received together with a gradient send
        grads_in: dict = {}  # gradients already received together with an activation send
        losses: List[float] = []
        self.peak_alive = 0
        nxt, prv = self.rank + 1, self.rank - 1
        for pos, (kind, i) in enumerate(order):
            follow = order[pos + 1] if pos + 1 < len(order) else None
            if kind == "F":
                if self.first:
                    x = micro_batches[i].to(self.device)
                else:
                    x = acts_in.pop(i, None)
                    if x is None:
                        x = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
                        _batch([], [(x, prv)], self.group)
                    x.requires_grad_(True)
                y = self.module(x)
                if self.last:
                    loss = loss_fn(y, targets[i].to(self.device)) / micro
                    losses.append(float(loss.detach()) * micro)
                    outputs[i] = loss
                else:
                    outputs[i] = y
                    out = y.detach().contiguous()
                    if follow is not None and follow[0] == "B":
                        # steady state: the activation goes out and the next gradient comes in as one group
                        g = torch.empty_like(outputs[follow[1]])
                        _batch([(out, nxt)], [(g, nxt)], self.group)
                        grads_in[follow[1]] = g
                    else:
                        _batch([(out, nxt)], [], self.group)
                inputs[i] = x
                self.peak_alive = max(self.peak_alive, len(outputs))
            else:
                y = outputs.pop(i)
                x = inputs.pop(i)
                if self.last:
                    y.backward()
                else:
                    g = grads_in.pop(i, None)
                    if g is None:
                        g = torch.empty_like(y)
                        _batch([], [(g, nxt)], self.group)
                    torch.autograd.backward(y, g)
                if not self.first:
                    gx = x.grad.contiguous()
                    if follow is not None and follow[0] == "F":
                        xn = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
                        _batch([(gx, prv)], [(xn, prv)], self.group)
                        acts_in[follow[1]] = xn
                    else:
                        _batch([(gx, prv)], [], self.group)
        return losses
