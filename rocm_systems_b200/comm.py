"""Python face of the native communicator (``libb200coll.so``) for torch CUDA tensors.

One :class:`Communicator` per process and GPU. Collectives are enqueued on the current torch CUDA
stream (or the one given) and return at once, like their C counterparts
(``csrc/include/b200coll/nccl.h``).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

from . import _lib

_DTYPES = {
    torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6, torch.float32: 7,
    torch.float64: 8, torch.bfloat16: 9,
}
if hasattr(torch, "uint32"):
    _DTYPES[torch.uint32] = 3
if hasattr(torch, "uint64"):
    _DTYPES[torch.uint64] = 5
if hasattr(torch, "float8_e4m3fn"):
    _DTYPES[torch.float8_e4m3fn] = 10
    _DTYPES[torch.float8_e5m2] = 11

OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}

LAUNCHES = 0  # collective kernels enqueued through this module (bench.py reports it)


def _k(rc: int, where: str) -> None:
    global LAUNCHES
    _lib.check(rc, where)
    LAUNCHES += 1


def nccl_dtype(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"dtype {dt} has no collective element type") from None


def get_unique_id() -> bytes:
    """Make a rendezvous id (starts the root service in this process). Share it with every rank."""
    lib = _lib.load()
    uid = _lib.UniqueId()
    _lib.check(lib.ncclGetUniqueId(ctypes.byref(uid)), "ncclGetUniqueId")
    return ctypes.string_at(ctypes.addressof(uid), _lib.NCCL_UNIQUE_ID_BYTES)


def _stream(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


class SymmetricTensor:
    """A tensor view over memory that every rank of a communicator maps (``b200collSymAlloc``)."""

    def __init__(self, comm: "Communicator", ptr: int, nbytes: int):
        self.comm, self.ptr, self.nbytes = comm, ptr, nbytes

    def tensor(self, shape: Sequence[int], dtype: torch.dtype, offset_bytes: int = 0, peer: Optional[int] = None) -> torch.Tensor:
        """View (part of) the allocation as a tensor; ``peer`` selects another rank's copy."""
        base = self.ptr if peer is None else self.comm.peer_ptr(self.ptr, peer)
        return _tensor_from_ptr(base + offset_bytes, shape, dtype, self.comm.device)

    def multicast_ptr(self) -> int:
        return self.comm.multicast_ptr(self.ptr)

    def free(self) -> None:
        if self.ptr:
            self.comm.sym_free(self.ptr)
            self.ptr = 0


class _CudaArray:
    """Minimal __cuda_array_interface__ carrier so torch can wrap foreign device memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _tensor_from_ptr(ptr: int, shape: Sequence[int], dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    with torch.cuda.device(device):
        raw = torch.as_tensor(_CudaArray(ptr, max(nbytes, 1)), device=device)
    return raw[:nbytes].view(dtype).view(*shape)


class Communicator:
    """One rank of a communicator of the native library: a method per collective of the C API (rccl.h:655-1051 for the
    semantics: in-place rules, grouped send/recv, PreMulSum operators, split colours), symmetric allocations, host-side
    barrier / all-gather over the rendezvous network, and the per-collective trace records. Tensors are passed by
    address on the current (or given) CUDA stream; nothing here synchronises the device unless it says so.
    """

    def __init__(self, rank: int, nranks: int, unique_id: bytes, device: Optional[int] = None,
                 min_ctas: Optional[int] = None, max_ctas: Optional[int] = None):
        self._lib = _lib.load()
        if device is None:
            device = torch.cuda.current_device()
        self.device = torch.device("cuda", device)
        self.rank, self.nranks = rank, nranks
        uid = _lib.UniqueId()
        ctypes.memmove(ctypes.addressof(uid), unique_id, _lib.NCCL_UNIQUE_ID_BYTES)
        self._h = ctypes.c_void_p()
        cfg = _lib.Config.default()
        if min_ctas:
            cfg.minCTAs = min_ctas
        if max_ctas:
            cfg.maxCTAs = max_ctas
        with torch.cuda.device(self.device):
            torch.cuda.init()
            torch.zeros(1, device=self.device)  # make the primary context current
            _lib.check(self._lib.ncclCommInitRankConfig(ctypes.byref(self._h), nranks, uid, rank, ctypes.byref(cfg)), "ncclCommInitRank")

    # ---- lifetime -----------------------------------------------------------------------------
    def destroy(self) -> None:
        if self._h:
            _lib.check(self._lib.ncclCommDestroy(self._h), "ncclCommDestroy")
            self._h = ctypes.c_void_p()

    def abort(self) -> None:
        if self._h:
            self._lib.ncclCommAbort(self._h)
            self._h = ctypes.c_void_p()

    def split(self, color: int, key: int) -> Optional["Communicator"]:
        new = ctypes.c_void_p()
        _lib.check(self._lib.ncclCommSplit(self._h, color, key, ctypes.byref(new), None), "ncclCommSplit")
        if not new:
            return None
        c = object.__new__(Communicator)
        c._lib, c._h, c.device = self._lib, new, self.device
        r, n = ctypes.c_int(), ctypes.c_int()
        self._lib.ncclCommUserRank(new, ctypes.byref(r))
        self._lib.ncclCommCount(new, ctypes.byref(n))
        c.rank, c.nranks = r.value, n.value
        return c

    def async_error(self) -> int:
        e = ctypes.c_int()
        _lib.check(self._lib.ncclCommGetAsyncError(self._h, ctypes.byref(e)), "ncclCommGetAsyncError")
        return e.value

    def last_error(self) -> str:
        return self._lib.ncclGetLastError(self._h).decode()

    @property
    def nvls(self) -> bool:
        """True when the communicator has an NVSwitch multicast alias of its workspace."""
        return bool(self._lib.b200collCommCaps(self._h) & 1)

    def _test_wait_timeout(self, timeout_ms: int = 500, stream=None) -> None:
        _lib.check(self._lib.b200collTestWaitTimeout(self._h, timeout_ms, _stream(stream)), "b200collTestWaitTimeout")

    @property
    def handle(self) -> int:
        return self._h.value

    # ---- collectives --------------------------------------------------------------------------
    def all_reduce(self, send: torch.Tensor, recv: Optional[torch.Tensor] = None, op="sum", stream=None) -> torch.Tensor:
        recv = send if recv is None else recv
        opv = OPS[op] if isinstance(op, str) else int(op)
        _k(self._lib.ncclAllReduce(send.data_ptr(), recv.data_ptr(), send.numel(), nccl_dtype(send.dtype), opv, self._h, _stream(stream)), "ncclAllReduce")
        return recv

    def reduce_scatter(self, send: torch.Tensor, recv: torch.Tensor, op="sum", stream=None) -> torch.Tensor:
        opv = OPS[op] if isinstance(op, str) else int(op)
        assert send.numel() == recv.numel() * self.nranks
        _k(self._lib.ncclReduceScatter(send.data_ptr(), recv.data_ptr(), recv.numel(), nccl_dtype(send.dtype), opv, self._h, _stream(stream)), "ncclReduceScatter")
        return recv

    def all_gather(self, send: torch.Tensor, recv: torch.Tensor, stream=None) -> torch.Tensor:
        assert recv.numel() == send.numel() * self.nranks
        _k(self._lib.ncclAllGather(send.data_ptr(), recv.data_ptr(), send.numel(), nccl_dtype(send.dtype), self._h, _stream(stream)), "ncclAllGather")
        return recv

    def broadcast(self, send: torch.Tensor, recv: Optional[torch.Tensor] = None, root: int = 0, stream=None) -> torch.Tensor:
        recv = send if recv is None else recv
        _k(self._lib.ncclBroadcast(send.data_ptr(), recv.data_ptr(), recv.numel(), nccl_dtype(recv.dtype), root, self._h, _stream(stream)), "ncclBroadcast")
        return recv

    def reduce(self, send: torch.Tensor, recv: Optional[torch.Tensor], root: int = 0, op="sum", stream=None):
        opv = OPS[op] if isinstance(op, str) else int(op)
        rp = recv.data_ptr() if recv is not None else None
        _k(self._lib.ncclReduce(send.data_ptr(), rp, send.numel(), nccl_dtype(send.dtype), opv, root, self._h, _stream(stream)), "ncclReduce")
        return recv

    def all_to_all(self, send: torch.Tensor, recv: torch.Tensor, stream=None) -> torch.Tensor:
        assert send.numel() == recv.numel() and send.numel() % self.nranks == 0
        _k(self._lib.ncclAllToAll(send.data_ptr(), recv.data_ptr(), send.numel() // self.nranks, nccl_dtype(send.dtype), self._h, _stream(stream)), "ncclAllToAll")
        return recv

    def all_to_allv(self, send, sendcounts, sdispls, recv, recvcounts, rdispls, stream=None):
        n = self.nranks
        arr = lambda v: (ctypes.c_size_t * n)(*[int(x) for x in v])
        _k(self._lib.ncclAllToAllv(send.data_ptr(), arr(sendcounts), arr(sdispls), recv.data_ptr(), arr(recvcounts), arr(rdispls),
                                           nccl_dtype(send.dtype), self._h, _stream(stream)), "ncclAllToAllv")
        return recv

    def gather(self, send, recv, root=0, stream=None):
        rp = recv.data_ptr() if recv is not None else None
        _k(self._lib.ncclGather(send.data_ptr(), rp, send.numel(), nccl_dtype(send.dtype), root, self._h, _stream(stream)), "ncclGather")
        return recv

    def scatter(self, send, recv, root=0, stream=None):
        sp = send.data_ptr() if send is not None else None
        _k(self._lib.ncclScatter(sp, recv.data_ptr(), recv.numel(), nccl_dtype(recv.dtype), root, self._h, _stream(stream)), "ncclScatter")
        return recv

    def send(self, t: torch.Tensor, peer: int, stream=None) -> None:
        _k(self._lib.ncclSend(t.data_ptr(), t.numel(), nccl_dtype(t.dtype), peer, self._h, _stream(stream)), "ncclSend")

    def recv(self, t: torch.Tensor, peer: int, stream=None) -> None:
        _k(self._lib.ncclRecv(t.data_ptr(), t.numel(), nccl_dtype(t.dtype), peer, self._h, _stream(stream)), "ncclRecv")

    def group_start(self) -> None:
        _lib.check(self._lib.ncclGroupStart(), "ncclGroupStart")

    def group_end(self) -> None:
        _lib.check(self._lib.ncclGroupEnd(), "ncclGroupEnd")

    def barrier(self, stream=None) -> None:
        _k(self._lib.b200collBarrier(self._h, _stream(stream)), "b200collBarrier")

    def host_barrier(self) -> None:
        _lib.check(self._lib.b200collHostBarrier(self._h), "b200collHostBarrier")

    def host_all_gather(self, data: bytes) -> list:
        n = len(data)
        out = ctypes.create_string_buffer(n * self.nranks)
        _lib.check(self._lib.b200collHostAllGather(self._h, data, out, n), "b200collHostAllGather")
        return [out.raw[i * n:(i + 1) * n] for i in range(self.nranks)]

    def premul_sum(self, scalar: float, dtype: torch.dtype) -> int:
        """Create a PreMulSum operator (host-immediate scalar); returns the op handle."""
        t = torch.tensor([scalar], dtype=dtype)
        buf = (ctypes.c_char * 8)()
        raw = t.view(torch.uint8).numpy().tobytes()
        ctypes.memmove(buf, raw, len(raw))
        op = ctypes.c_int()
        _lib.check(self._lib.ncclRedOpCreatePreMulSum(ctypes.byref(op), buf, nccl_dtype(dtype), 1, self._h), "ncclRedOpCreatePreMulSum")
        return op.value

    def premul_sum_device(self, scalar: torch.Tensor) -> int:
        """Create a PreMulSum operator whose scalar lives in device memory (a one-element tensor of the data type). The
        reducing kernel reads it when it runs, in stream order: the value may be produced by earlier work on the same
        stream, the call does not wait for the stream and can be captured in a graph. Keep the tensor alive until the
        operator is destroyed."""
        assert scalar.is_cuda and scalar.numel() == 1
        op = ctypes.c_int()
        _lib.check(self._lib.ncclRedOpCreatePreMulSum(ctypes.byref(op), ctypes.c_void_p(scalar.data_ptr()), nccl_dtype(scalar.dtype), 0, self._h),
                   "ncclRedOpCreatePreMulSum")
        return op.value

    def redop_destroy(self, op: int) -> None:
        _lib.check(self._lib.ncclRedOpDestroy(op, self._h), "ncclRedOpDestroy")

    # ---- symmetric memory ---------------------------------------------------------------------
    def sym_alloc(self, nbytes: int) -> SymmetricTensor:
        p = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self._lib.b200collSymAlloc(self._h, nbytes, ctypes.byref(p)), "b200collSymAlloc")
        return SymmetricTensor(self, p.value, nbytes)

    def sym_free(self, ptr: int) -> None:
        _lib.check(self._lib.b200collSymFree(self._h, ptr), "b200collSymFree")

    def peer_ptr(self, ptr: int, peer: int) -> int:
        out = ctypes.c_void_p()
        _lib.check(self._lib.b200collSymPeerPtr(self._h, ptr, peer, ctypes.byref(out)), "b200collSymPeerPtr")
        return out.value

    def multicast_ptr(self, ptr: int) -> int:
        out = ctypes.c_void_p()
        _lib.check(self._lib.b200collSymMulticastPtr(self._h, ptr, ctypes.byref(out)), "b200collSymMulticastPtr")
        return out.value or 0

    # ---- tracing --------------------------------------------------------------------------------
    def trace_enable(self, on: bool = True) -> None:
        _lib.check(self._lib.b200collTraceEnable(self._h, int(on)), "b200collTraceEnable")

    def trace_records(self) -> list:
        n = ctypes.c_size_t()
        _lib.check(self._lib.b200collTraceGet(self._h, None, 0, ctypes.byref(n)), "b200collTraceGet")
        if n.value == 0:
            return []
        arr = (_lib.TraceRecord * n.value)()
        _lib.check(self._lib.b200collTraceGet(self._h, arr, n.value, ctypes.byref(n)), "b200collTraceGet")
        out = []
        for r in arr:
            out.append({f[0]: getattr(r, f[0]) for f in _lib.TraceRecord._fields_} | {"api": self._lib.b200collApiName(r.opId).decode()})
        return out

    def trace_clear(self) -> None:
        _lib.check(self._lib.b200collTraceClear(self._h), "b200collTraceClear")

    def trace_write(self, path: str, fmt: str = "csv") -> None:
        _lib.check(self._lib.b200collTraceWrite(self._h, path.encode(), fmt.encode()), "b200collTraceWrite")


def init_from_env(device: Optional[int] = None, port_offset: int = 17, min_ctas: Optional[int] = None, max_ctas: Optional[int] = None) -> Communicator:
    """Build a communicator from torchrun-style variables (RANK, WORLD_SIZE, LOCAL_RANK,
    MASTER_ADDR, MASTER_PORT): rank 0 makes the id and shares it through a TCPStore. ``max_ctas`` caps the CTAs of its
    collectives (a communicator whose collectives overlap GEMMs wants fewer than one that runs alone); a second
    communicator of the same job needs another ``port_offset``."""
    from torch.distributed import TCPStore

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if device is None:
        device = local
    torch.cuda.set_device(device)
    from .utils import affinity

    if affinity.wanted():
        affinity.pin_to_gpu(device)   # B200COLL_CPU_AFFINITY=1: run on the CPUs next to this rank's GPU
    if world == 1:
        return Communicator(0, 1, get_unique_id(), device, min_ctas, max_ctas)
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500")) + port_offset
    store = TCPStore(addr, port, world, is_master=(rank == 0), wait_for_workers=False)
    if rank == 0:
        uid = get_unique_id()
        store.set("b200coll_uid", uid)
    else:
        uid = store.get("b200coll_uid")
    comm = Communicator(rank, world, uid, device, min_ctas, max_ctas)
    comm._store = store  # keep the store alive as long as the communicator
    return comm
