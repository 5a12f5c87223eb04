"""The slice of the ``Communicator`` interface the FSDP engine uses, served by stock NCCL through
``torch.distributed``. It exists for one purpose: a control run of the same trainer with the
library collectives swapped for NCCL's (``bench.py --collectives nccl``), so "tokens/s with this
package's collectives vs with NCCL's" compares nothing but the collectives.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

_OPS = {"sum": dist.ReduceOp.SUM, "avg": dist.ReduceOp.AVG, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "prod": dist.ReduceOp.PRODUCT}


class NcclComm:
    """The collectives the FSDP engine calls, on stock NCCL through ``torch.distributed`` (control runs only)."""

    def __init__(self, group=None):
        if not dist.is_initialized():
            raise RuntimeError("init torch.distributed with backend='nccl' first")
        self.group = group
        self.rank = dist.get_rank(group)
        self.nranks = dist.get_world_size(group)
        self.device = torch.device("cuda", torch.cuda.current_device())

    def _on(self, stream, fn) -> None:
        # NCCL work is enqueued on torch's internal stream, ordered after the current stream at the
        # call and before it at wait(): running the call under `stream` gives the engine's ordering.
        if stream is None:
            fn().wait()
            return
        with torch.cuda.stream(stream):
            fn().wait()

    def all_gather(self, send: torch.Tensor, recv: torch.Tensor, stream=None) -> torch.Tensor:
        self._on(stream, lambda: dist.all_gather_into_tensor(recv, send, group=self.group, async_op=True))
        return recv

    def reduce_scatter(self, send: torch.Tensor, recv: torch.Tensor, op="sum", stream=None) -> torch.Tensor:
        self._on(stream, lambda: dist.reduce_scatter_tensor(recv, send, op=_OPS[op], group=self.group, async_op=True))
        return recv

    def all_reduce(self, send: torch.Tensor, recv=None, op="sum", stream=None) -> torch.Tensor:
        out = send if recv is None else recv.copy_(send)
        self._on(stream, lambda: dist.all_reduce(out, op=_OPS[op], group=self.group, async_op=True))
        return out

    def host_barrier(self) -> None:
        dist.barrier(group=self.group)

    def host_all_gather(self, data: bytes) -> list:
        out = [None] * self.nranks
        dist.all_gather_object(out, data, group=self.group)
        return out

    def async_error(self) -> int:
        return 0

    def last_error(self) -> str:
        return ""

    def destroy(self) -> None:
        pass
