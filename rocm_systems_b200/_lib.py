"""ctypes loader for ``lib/libb200coll.so`` (the native collective library).

The library is built in-tree by :mod:`rocm_systems_b200.utils.build`; nothing here falls back to
another implementation. If the shared object is missing the import fails with the build command.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "lib" / "libb200coll.so"

NCCL_UNIQUE_ID_BYTES = 128


class UniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_char * NCCL_UNIQUE_ID_BYTES)]


class TraceRecord(ctypes.Structure):
    _fields_ = [
        ("correlationId", ctypes.c_uint64), ("opId", ctypes.c_int32), ("dtype", ctypes.c_int32),
        ("count", ctypes.c_uint64), ("bytes", ctypes.c_uint64), ("algo", ctypes.c_int32), ("ctas", ctypes.c_int32),
        ("hostBeginNs", ctypes.c_uint64), ("hostEndNs", ctypes.c_uint64), ("devBeginNs", ctypes.c_uint64),
        ("devEndNs", ctypes.c_uint64),
    ]


class Config(ctypes.Structure):
    _fields_ = [
        ("size", ctypes.c_size_t), ("magic", ctypes.c_uint), ("version", ctypes.c_uint), ("blocking", ctypes.c_int),
        ("cgaClusterSize", ctypes.c_int), ("minCTAs", ctypes.c_int), ("maxCTAs", ctypes.c_int),
        ("netName", ctypes.c_char_p), ("splitShare", ctypes.c_int),
    ]

    @classmethod
    def default(cls) -> "Config":
        undef = -(2 ** 31)
        return cls(ctypes.sizeof(cls), 0xCAFEBEEF, 22005, undef, undef, undef, undef, None, undef)


_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m rocm_systems_b200.utils.build` "
            "(needs nvcc; no GPU required to build)")
    lib = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_GLOBAL)
    vp, sz, i32 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    lib.ncclGetErrorString.restype = ctypes.c_char_p
    lib.ncclGetLastError.restype = ctypes.c_char_p
    lib.ncclGetLastError.argtypes = [vp]
    lib.b200collLastError.restype = ctypes.c_char_p
    lib.b200collApiName.restype = ctypes.c_char_p
    lib.ncclGetUniqueId.argtypes = [ctypes.POINTER(UniqueId)]
    lib.ncclCommInitRank.argtypes = [ctypes.POINTER(vp), i32, UniqueId, i32]
    lib.ncclCommInitRankConfig.argtypes = [ctypes.POINTER(vp), i32, UniqueId, i32, ctypes.POINTER(Config)]
    lib.ncclCommSplit.argtypes = [vp, i32, i32, ctypes.POINTER(vp), ctypes.POINTER(Config)]
    for name in ("ncclCommDestroy", "ncclCommAbort", "ncclCommFinalize"):
        getattr(lib, name).argtypes = [vp]
    lib.ncclCommGetAsyncError.argtypes = [vp, ctypes.POINTER(i32)]
    lib.ncclAllReduce.argtypes = [vp, vp, sz, i32, i32, vp, vp]
    lib.ncclReduceScatter.argtypes = [vp, vp, sz, i32, i32, vp, vp]
    lib.ncclAllGather.argtypes = [vp, vp, sz, i32, vp, vp]
    lib.ncclBroadcast.argtypes = [vp, vp, sz, i32, i32, vp, vp]
    lib.ncclReduce.argtypes = [vp, vp, sz, i32, i32, i32, vp, vp]
    lib.ncclAllToAll.argtypes = [vp, vp, sz, i32, vp, vp]
    lib.ncclAllToAllv.argtypes = [vp, ctypes.POINTER(sz), ctypes.POINTER(sz), vp, ctypes.POINTER(sz), ctypes.POINTER(sz), i32, vp, vp]
    lib.ncclGather.argtypes = [vp, vp, sz, i32, i32, vp, vp]
    lib.ncclScatter.argtypes = [vp, vp, sz, i32, i32, vp, vp]
    lib.ncclSend.argtypes = [vp, sz, i32, i32, vp, vp]
    lib.ncclRecv.argtypes = [vp, sz, i32, i32, vp, vp]
    lib.ncclMemAlloc.argtypes = [ctypes.POINTER(vp), sz]
    lib.ncclMemFree.argtypes = [vp]
    lib.ncclCommRegister.argtypes = [vp, vp, sz, ctypes.POINTER(vp)]
    lib.ncclCommDeregister.argtypes = [vp, vp]
    lib.ncclRedOpCreatePreMulSum.argtypes = [ctypes.POINTER(i32), vp, i32, i32, vp]
    lib.ncclRedOpDestroy.argtypes = [i32, vp]
    lib.b200collSymAlloc.argtypes = [vp, sz, ctypes.POINTER(vp)]
    lib.b200collSymFree.argtypes = [vp, vp]
    lib.b200collSymPeerPtr.argtypes = [vp, vp, i32, ctypes.POINTER(vp)]
    lib.b200collSymMulticastPtr.argtypes = [vp, vp, ctypes.POINTER(vp)]
    lib.b200collHostBarrier.argtypes = [vp]
    lib.b200collHostAllGather.argtypes = [vp, vp, vp, sz]
    lib.b200collBarrier.argtypes = [vp, vp]
    lib.b200collTraceEnable.argtypes = [vp, i32]
    lib.b200collTraceGet.argtypes = [vp, ctypes.POINTER(TraceRecord), sz, ctypes.POINTER(sz)]
    lib.b200collTraceClear.argtypes = [vp]
    lib.b200collTraceWrite.argtypes = [vp, ctypes.c_char_p, ctypes.c_char_p]
    lib.b200collBootCreate.argtypes = [ctypes.POINTER(UniqueId), i32, i32, ctypes.POINTER(vp)]
    lib.b200collBootAllGather.argtypes = [vp, vp, vp, sz]
    lib.b200collBootBarrier.argtypes = [vp]
    lib.b200collBootSendFd.argtypes = [vp, i32, i32, ctypes.c_uint32]
    lib.b200collBootRecvFd.argtypes = [vp, i32, ctypes.c_uint32, ctypes.POINTER(i32)]
    lib.b200collBootPeerFailed.argtypes = [vp]
    lib.b200collBootClose.argtypes = [vp, i32]
    lib.mscclLoadAlgo.argtypes = [ctypes.c_char_p, ctypes.POINTER(i32), i32]
    lib.mscclUnloadAlgo.argtypes = [i32]
    lib.mscclRunAlgo.argtypes = [vp, vp, vp, vp, vp, vp, sz, i32, i32, i32, i32, i32, vp, vp]
    lib.b200collGetApiTable.restype = vp
    lib.b200collTestWaitTimeout.argtypes = [vp, i32, vp]
    lib.b200collCommCaps.argtypes = [vp]
    _lib = lib
    return lib


class B200CollError(RuntimeError):
    def __init__(self, code: int, where: str):
        lib = load()
        msg = lib.ncclGetErrorString(code).decode()
        detail = lib.b200collLastError().decode()
        super().__init__(f"{where}: {msg} [{code}] {detail}")
        self.code = code


def check(code: int, where: str = "b200coll") -> None:
    if code != 0:
        raise B200CollError(code, where)
