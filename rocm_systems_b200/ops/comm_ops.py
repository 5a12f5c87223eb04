"""Fused compute+communication ops on torch tensors (``csrc/include/b200coll/fused.h``)."""
from __future__ import annotations

import ctypes

import torch

from .. import _lib
from . import train_ops

_done = False


def _lib_fused():
    global _done
    lib = _lib.load()
    if not _done:
        vp = ctypes.c_void_p
        lib.b200collReduceScatterCast.argtypes = [vp, vp, vp, ctypes.c_size_t, ctypes.c_float, vp]
        _done = True
    return lib


def reduce_scatter_cast(comm, send_bf16: torch.Tensor, recv_f32: torch.Tensor, scale: float, stream=None) -> torch.Tensor:
    """``recv = scale * sum_over_ranks(send)[rank slice]`` with fp32 accumulation, one kernel."""
    assert send_bf16.dtype == torch.bfloat16 and recv_f32.dtype == torch.float32
    assert send_bf16.is_contiguous() and recv_f32.is_contiguous()
    assert send_bf16.numel() == recv_f32.numel() * comm.nranks
    s = (stream or torch.cuda.current_stream()).cuda_stream
    _lib.check(_lib_fused().b200collReduceScatterCast(comm.handle, send_bf16.data_ptr(), recv_f32.data_ptr(), recv_f32.numel(), scale, s),
               "b200collReduceScatterCast")
    train_ops.LAUNCHES += 1
    return recv_f32
