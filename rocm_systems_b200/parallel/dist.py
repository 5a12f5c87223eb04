"""``torch.distributed`` integration: registers the ``b200coll`` backend (the native library's
collectives behind a ``c10d::Backend``, csrc/torch/pg_b200.cpp) and offers an
``init_process_group`` that routes CUDA tensors to it and CPU tensors to gloo.
"""
from __future__ import annotations

import datetime
from typing import Optional

import torch
import torch.distributed as dist

BACKEND_NAME = "b200coll"
_registered = False


def _load_ext():
    try:
        from .. import _C  # noqa: F401
    except ImportError as e:  # pragma: no cover - build problem, say how to fix it
        raise ImportError(
            "rocm_systems_b200._C (the c10d backend extension) is not built: run "
            "`python -m rocm_systems_b200.utils.build`") from e
    return _C


def register_backend() -> None:
    """Make ``backend="b200coll"`` (and ``"cpu:gloo,cuda:b200coll"``) known to torch.distributed."""
    global _registered
    if _registered:
        return
    ext = _load_ext()

    def _create(store, rank, size, timeout):
        return ext.create_backend(store, rank, size, timeout)

    dist.Backend.register_backend(BACKEND_NAME, _create, devices=["cuda"])
    _registered = True


def init_process_group(rank: Optional[int] = None, world_size: Optional[int] = None, init_method: Optional[str] = None,
                       timeout: Optional[datetime.timedelta] = None, device_id: Optional[torch.device] = None):
    """``dist.init_process_group`` with CUDA collectives on b200coll and CPU collectives on gloo.

    Reads RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT like torchrun sets them unless given.
    """
    register_backend()
    kw = {}
    if rank is not None:
        kw["rank"] = rank
    if world_size is not None:
        kw["world_size"] = world_size
    if init_method is not None:
        kw["init_method"] = init_method
    if timeout is not None:
        kw["timeout"] = timeout
    if device_id is not None and torch.cuda.is_available():
        torch.cuda.set_device(device_id)
    from ..utils import affinity

    if torch.cuda.is_available() and affinity.wanted():   # B200COLL_CPU_AFFINITY=1: run on the CPUs next to this rank's GPU
        affinity.pin_to_gpu(torch.cuda.current_device())
    dist.init_process_group(backend=f"cpu:gloo,cuda:{BACKEND_NAME}", **kw)
    return dist.group.WORLD
