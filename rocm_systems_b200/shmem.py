"""Python face of the OpenSHMEM-style layer (csrc/include/b200coll/shmem.h): a symmetric heap on top
of a communicator, stream-ordered put / get / put-with-signal / wait / barrier issued from the
host, and access to the device context that kernels of an extension pass to ``shmem_device.cuh``.

    sh = Shmem(comm, heap_bytes=256 << 20)
    buf = sh.malloc_tensor((1 << 20,), torch.float32)       # same offset on every PE
    sh.barrier_all()
    sh.put(buf, src, pe=(sh.my_pe + 1) % sh.n_pes)
    sh.barrier_all()

The reference only consumes such a layer (rocSHMEM is outside its snapshot); the calls follow the
OpenSHMEM names the device header uses.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from . import _lib
from .comm import _tensor_from_ptr

CMP_EQ, CMP_NE, CMP_GT, CMP_GE, CMP_LT, CMP_LE = 0, 1, 2, 3, 4, 5
SIGNAL_SET, SIGNAL_ADD = 0, 1
_sigs = False


def _l():
    global _sigs
    lib = _lib.load()
    if not _sigs:
        vp, sz, i32, u64 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_ulonglong
        lib.b200shmem_init.argtypes = [vp, sz, ctypes.POINTER(vp)]
        lib.b200shmem_finalize.argtypes = [vp]
        lib.b200shmem_my_pe.argtypes = [vp]
        lib.b200shmem_n_pes.argtypes = [vp]
        lib.b200shmem_malloc.argtypes = [vp, sz]
        lib.b200shmem_malloc.restype = vp
        lib.b200shmem_align.argtypes = [vp, sz, sz]
        lib.b200shmem_align.restype = vp
        lib.b200shmem_free.argtypes = [vp, vp]
        lib.b200shmem_ptr.argtypes = [vp, vp, i32]
        lib.b200shmem_ptr.restype = vp
        lib.b200shmem_mc_ptr.argtypes = [vp, vp]
        lib.b200shmem_mc_ptr.restype = vp
        lib.b200shmem_putmem_on_stream.argtypes = [vp, vp, vp, sz, i32, vp]
        lib.b200shmem_getmem_on_stream.argtypes = [vp, vp, vp, sz, i32, vp]
        lib.b200shmem_putmem_signal_on_stream.argtypes = [vp, vp, vp, sz, vp, u64, i32, i32, vp]
        lib.b200shmem_signal_wait_until_on_stream.argtypes = [vp, vp, i32, u64, vp]
        lib.b200shmem_barrier_all_on_stream.argtypes = [vp, vp]
        lib.b200shmem_take_status.argtypes = [vp]
        lib.b200shmem_putmem_dma_on_stream.argtypes = [vp, vp, vp, sz, i32, i32, vp]
        lib.b200shmem_getmem_dma_on_stream.argtypes = [vp, vp, vp, sz, i32, i32, vp]
        lib.b200shmem_putmem_signal_dma_on_stream.argtypes = [vp, vp, vp, sz, vp, u64, i32, i32, i32, vp]
        lib.b200shmem_dma_plan.argtypes = [sz, i32, ctypes.POINTER(sz), ctypes.POINTER(sz)]
        lib.b200shmem_dma_engines.argtypes = [vp]
        tp = ctypes.POINTER(Team)
        lib.b200shmem_team_world.argtypes = [vp, tp]
        lib.b200shmem_team_split_strided.argtypes = [vp, tp, i32, i32, i32, tp]
        lib.b200shmem_team_translate_pe.argtypes = [tp, i32, tp]
        lib.b200shmem_team_sync_on_stream.argtypes = [vp, tp, vp]
        _sigs = True
    return lib


class Team(ctypes.Structure):
    """``b200shmem_team_t``: the PEs ``start + i * stride`` for ``i < size``; ``idx`` is this PE's index in it (-1: not a
    member). Kernels take it by value next to the device context."""
    _fields_ = [("start", ctypes.c_int), ("stride", ctypes.c_int), ("size", ctypes.c_int), ("idx", ctypes.c_int),
                ("sync_flags", ctypes.c_void_p), ("sync_epoch", ctypes.c_void_p)]

    def pes(self) -> list:
        return [self.start + i * self.stride for i in range(self.size)]


def _stream(stream) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def dma_plan(nbytes: int, gang: int = 0) -> list[tuple[int, int]]:
    """(offset, length) of the parts a copy-engine transfer of ``nbytes`` is cut into. Needs no GPU."""
    lib = _l()
    offs, lens = (ctypes.c_size_t * 8)(), (ctypes.c_size_t * 8)()
    n = lib.b200shmem_dma_plan(nbytes, gang, offs, lens)
    return [(int(offs[i]), int(lens[i])) for i in range(n)]


class Shmem:
    """A symmetric heap on top of a communicator and the host-initiated, stream-ordered operations on it.
    Every PE must allocate in the same order; waits are bounded and report through ``take_status``.
    """

    def __init__(self, comm, heap_bytes: int = 64 << 20):
        self.comm = comm
        self.lib = _l()
        self._ctx = ctypes.c_void_p()
        _lib.check(self.lib.b200shmem_init(comm.handle, heap_bytes, ctypes.byref(self._ctx)), "b200shmem_init")
        self.my_pe = int(self.lib.b200shmem_my_pe(self._ctx))
        self.n_pes = int(self.lib.b200shmem_n_pes(self._ctx))

    @property
    def handle(self) -> int:
        return self._ctx.value

    def finalize(self) -> None:
        if self._ctx:
            torch.cuda.synchronize()
            _lib.check(self.lib.b200shmem_finalize(self._ctx), "b200shmem_finalize")
            self._ctx = ctypes.c_void_p()

    # ---- symmetric heap ----
    def malloc(self, nbytes: int, alignment: int = 0) -> int:
        ptr = self.lib.b200shmem_align(self._ctx, alignment, nbytes) if alignment else self.lib.b200shmem_malloc(self._ctx, nbytes)
        if not ptr:
            raise MemoryError(f"symmetric heap cannot hold {nbytes} more bytes")
        return int(ptr)

    def free(self, ptr: int) -> None:
        self.lib.b200shmem_free(self._ctx, ptr)

    def malloc_tensor(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """A tensor in the symmetric heap (same offset on every PE when every PE allocates in the
        same order). Free it with ``free(t.data_ptr())`` once no PE uses it."""
        n = 1
        for s in shape:
            n *= int(s)
        ptr = self.malloc(max(16, n * torch.empty((), dtype=dtype).element_size()), 256)
        return _tensor_from_ptr(ptr, tuple(shape), dtype, self.comm.device)

    def peer_ptr(self, ptr: int, pe: int) -> int:
        """The address under which PE ``pe``'s copy of a symmetric object is mapped here (load/store-able)."""
        return int(self.lib.b200shmem_ptr(self._ctx, ptr, pe) or 0)

    def peer_tensor(self, t: torch.Tensor, pe: int) -> torch.Tensor:
        return _tensor_from_ptr(self.peer_ptr(t.data_ptr(), pe), tuple(t.shape), t.dtype, self.comm.device)

    def multicast_ptr(self, ptr: int) -> int:
        return int(self.lib.b200shmem_mc_ptr(self._ctx, ptr) or 0)

    # ---- stream-ordered operations ----
    def put(self, dest: torch.Tensor, source: torch.Tensor, pe: int, stream=None) -> None:
        """Copy ``source`` (local) into PE ``pe``'s copy of the symmetric tensor ``dest``."""
        nbytes = source.numel() * source.element_size()
        _lib.check(self.lib.b200shmem_putmem_on_stream(self._ctx, dest.data_ptr(), source.data_ptr(), nbytes, pe, _stream(stream)), "putmem")

    def get(self, dest: torch.Tensor, source: torch.Tensor, pe: int, stream=None) -> None:
        """Copy PE ``pe``'s copy of the symmetric tensor ``source`` into ``dest`` (local)."""
        nbytes = dest.numel() * dest.element_size()
        _lib.check(self.lib.b200shmem_getmem_on_stream(self._ctx, dest.data_ptr(), source.data_ptr(), nbytes, pe, _stream(stream)), "getmem")

    def put_signal(self, dest: torch.Tensor, source: torch.Tensor, sig: torch.Tensor, value: int, pe: int, op: int = SIGNAL_SET, stream=None) -> None:
        nbytes = source.numel() * source.element_size()
        _lib.check(self.lib.b200shmem_putmem_signal_on_stream(self._ctx, dest.data_ptr(), source.data_ptr(), nbytes, sig.data_ptr(), value, op, pe,
                                                              _stream(stream)), "putmem_signal")

    # ---- the same by copy engine: no SM takes part, large transfers are split over `gang` engines ----
    def put_dma(self, dest: torch.Tensor, source: torch.Tensor, pe: int, gang: int = 0, stream=None) -> None:
        nbytes = source.numel() * source.element_size()
        _lib.check(self.lib.b200shmem_putmem_dma_on_stream(self._ctx, dest.data_ptr(), source.data_ptr(), nbytes, pe, gang, _stream(stream)), "putmem_dma")

    def get_dma(self, dest: torch.Tensor, source: torch.Tensor, pe: int, gang: int = 0, stream=None) -> None:
        nbytes = dest.numel() * dest.element_size()
        _lib.check(self.lib.b200shmem_getmem_dma_on_stream(self._ctx, dest.data_ptr(), source.data_ptr(), nbytes, pe, gang, _stream(stream)), "getmem_dma")

    def put_signal_dma(self, dest: torch.Tensor, source: torch.Tensor, sig: torch.Tensor, value: int, pe: int, op: int = SIGNAL_SET, gang: int = 0,
                       stream=None) -> None:
        nbytes = source.numel() * source.element_size()
        _lib.check(self.lib.b200shmem_putmem_signal_dma_on_stream(self._ctx, dest.data_ptr(), source.data_ptr(), nbytes, sig.data_ptr(), value, op, pe,
                                                                  gang, _stream(stream)), "putmem_signal_dma")

    def dma_engines(self) -> int:
        return int(self.lib.b200shmem_dma_engines(self._ctx))

    def wait_until(self, sig: torch.Tensor, cmp: int, value: int, stream=None) -> None:
        """Bounded device-side wait on a local signal word; a wait that runs out shows in ``take_status``."""
        _lib.check(self.lib.b200shmem_signal_wait_until_on_stream(self._ctx, sig.data_ptr(), cmp, value, _stream(stream)), "signal_wait_until")

    def barrier_all(self, stream=None) -> None:
        _lib.check(self.lib.b200shmem_barrier_all_on_stream(self._ctx, _stream(stream)), "barrier_all")

    def take_status(self) -> int:
        return int(self.lib.b200shmem_take_status(self._ctx))

    # ---- teams ------------------------------------------------------------------------------------------------------
    def team_world(self) -> Team:
        t = Team()
        _lib.check(self.lib.b200shmem_team_world(self._ctx, ctypes.byref(t)), "team_world")
        return t

    def team_split_strided(self, parent, start: int, stride: int, size: int) -> Team:
        """The team of ``parent``'s members ``start, start + stride, ...`` (``size`` of them; ``parent=None``: all PEs).
        EVERY PE of the context must make the same split calls in the same order, members or not."""
        t = Team()
        _lib.check(self.lib.b200shmem_team_split_strided(self._ctx, ctypes.byref(parent) if parent is not None else None, start, stride, size,
                                                         ctypes.byref(t)), "team_split_strided")
        return t

    def team_translate_pe(self, src: Team, idx: int, dst: Team) -> int:
        return int(self.lib.b200shmem_team_translate_pe(ctypes.byref(src), idx, ctypes.byref(dst)))

    def team_sync(self, team: Team, stream=None) -> None:
        _lib.check(self.lib.b200shmem_team_sync_on_stream(self._ctx, ctypes.byref(team), _stream(stream)), "team_sync")
