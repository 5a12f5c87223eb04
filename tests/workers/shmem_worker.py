"""One rank of the device-initiated communication self-tests (put+signal ring, remote atomics)."""
import ctypes
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402

from rocm_systems_b200 import _lib  # noqa: E402
from rocm_systems_b200.comm import init_from_env  # noqa: E402


def main():
    comm = init_from_env()
    lib = _lib.load()
    vp = ctypes.c_void_p
    lib.b200shmem_init.argtypes = [vp, ctypes.c_size_t, ctypes.POINTER(vp)]
    lib.b200shmem_finalize.argtypes = [vp]
    lib.b200shmem_selftest_ring.argtypes = [vp, ctypes.c_size_t, ctypes.c_int, vp, ctypes.POINTER(ctypes.c_int)]
    lib.b200shmem_selftest_atomics.argtypes = [vp, ctypes.c_int, vp, ctypes.POINTER(ctypes.c_int)]
    lib.b200shmem_selftest_collectives.argtypes = [vp, ctypes.c_size_t, vp, ctypes.POINTER(ctypes.c_int)]
    lib.b200shmem_selftest_teams.argtypes = [vp, ctypes.c_size_t, vp, ctypes.POINTER(ctypes.c_int)]
    lib.b200shmem_take_status.argtypes = [vp]
    lib.b200shmem_malloc.argtypes = [vp, ctypes.c_size_t]
    lib.b200shmem_malloc.restype = vp
    lib.b200shmem_free.argtypes = [vp, vp]
    lib.b200shmem_putmem_signal_on_stream.argtypes = [vp, vp, vp, ctypes.c_size_t, vp, ctypes.c_ulonglong, ctypes.c_int, ctypes.c_int, vp]
    lib.b200shmem_signal_wait_until_on_stream.argtypes = [vp, vp, ctypes.c_int, ctypes.c_ulonglong, vp]
    lib.b200shmem_barrier_all_on_stream.argtypes = [vp, vp]
    ctx = vp()
    _lib.check(lib.b200shmem_init(comm.handle, 64 << 20, ctypes.byref(ctx)), "b200shmem_init")
    s = torch.cuda.current_stream().cuda_stream
    bad = []
    errs = ctypes.c_int(-1)
    _lib.check(lib.b200shmem_selftest_ring(ctx, 100003, 6, s, ctypes.byref(errs)), "selftest_ring")
    if errs.value != 0:
        bad.append(("ring", errs.value))
    _lib.check(lib.b200shmem_selftest_atomics(ctx, 101, s, ctypes.byref(errs)), "selftest_atomics")
    if errs.value != 0:
        bad.append(("atomics", errs.value))
    if "--collectives" in sys.argv:   # block-scope collectives, wait_until / test, strided put of the device API
        _lib.check(lib.b200shmem_selftest_collectives(ctx, 1000, s, ctypes.byref(errs)), "selftest_collectives")
        if errs.value != 0:
            bad.append(("collectives", errs.value))
        # the same collectives inside teams (even PEs, odd PEs, every second even PE), all teams at once
        _lib.check(lib.b200shmem_selftest_teams(ctx, 1000, s, ctypes.byref(errs)), "selftest_teams")
        if errs.value != 0:
            bad.append(("teams", errs.value))
    # host-initiated, stream-ordered put with signal to the right neighbour
    n, rank = comm.nranks, comm.rank
    count = 1 << 16
    buf = lib.b200shmem_malloc(ctx, count * 4)
    sig = lib.b200shmem_malloc(ctx, 256)
    from rocm_systems_b200.comm import _tensor_from_ptr

    dst = _tensor_from_ptr(buf, (count,), torch.int32, comm.device)
    sigt = _tensor_from_ptr(sig, (32,), torch.int64, comm.device)
    dst.zero_()
    sigt.zero_()
    _lib.check(lib.b200shmem_barrier_all_on_stream(ctx, s), "barrier_all")
    src = torch.arange(count, device=comm.device, dtype=torch.int32) + 1000 * rank
    _lib.check(lib.b200shmem_putmem_signal_on_stream(ctx, buf, src.data_ptr(), count * 4, sig, 7, 0, (rank + 1) % n, s), "putmem_signal")
    _lib.check(lib.b200shmem_signal_wait_until_on_stream(ctx, sig, 0, 7, s), "signal_wait")
    torch.cuda.synchronize()
    want = torch.arange(count, device=comm.device, dtype=torch.int32) + 1000 * ((rank - 1) % n)
    if not torch.equal(dst, want):
        bad.append(("host_put_signal", int((dst != want).sum())))
    st = lib.b200shmem_take_status(ctx)
    if st != 0:
        bad.append(("status", st))
    comm.host_barrier()
    lib.b200shmem_free(ctx, sig)
    lib.b200shmem_free(ctx, buf)
    flags = comm.host_all_gather(bytes([1 if bad else 0]))
    if bad:
        print(f"[rank {rank}] SHMEM FAILURES: {bad}", flush=True)
    elif rank == 0:
        print(f"shmem_worker OK on {n} PEs", flush=True)
    _lib.check(lib.b200shmem_finalize(ctx), "b200shmem_finalize")
    comm.destroy()
    sys.exit(1 if any(f[0] for f in flags) else 0)


if __name__ == "__main__":
    main()
