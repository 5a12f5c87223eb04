"""One rank of the copy-engine put / get / put+signal test: every PE sends a pattern to its right neighbour
through the Python wrapper, for sizes that take 1, 2 and 4 engines, and reads its left neighbour's source back."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402

from rocm_systems_b200 import shmem  # noqa: E402
from rocm_systems_b200.comm import init_from_env  # noqa: E402


def main():
    comm = init_from_env()
    n, rank = comm.nranks, comm.rank
    sh = shmem.Shmem(comm, heap_bytes=320 << 20)
    right, left = (rank + 1) % n, (rank - 1) % n
    bad = []
    sig = sh.malloc_tensor((32,), torch.int64)
    sig.zero_()
    round_no = 0
    for nbytes, gang in [(4096, 0), (1 << 20, 0), ((8 << 20) + 4096, 0), (64 << 20, 0), (3 << 20, 8)]:
        round_no += 1
        count = nbytes // 4
        dst = sh.malloc_tensor((count,), torch.int32)
        srcsym = sh.malloc_tensor((count,), torch.int32)
        dst.zero_()
        srcsym.copy_(torch.arange(count, device=comm.device, dtype=torch.int32) * 3 + rank)
        sh.barrier_all()
        src = torch.arange(count, device=comm.device, dtype=torch.int32) + 1000 * rank + round_no
        sh.put_signal_dma(dst, src, sig, round_no, right, gang=gang)
        sh.wait_until(sig, shmem.CMP_GE, round_no)
        torch.cuda.synchronize()
        want = torch.arange(count, device=comm.device, dtype=torch.int32) + 1000 * left + round_no
        if not torch.equal(dst, want):
            bad.append(("put_signal_dma", nbytes, int((dst != want).sum())))
        got = torch.empty(count, device=comm.device, dtype=torch.int32)
        sh.get_dma(got, srcsym, left, gang=gang)
        torch.cuda.synchronize()
        if not torch.equal(got, torch.arange(count, device=comm.device, dtype=torch.int32) * 3 + left):
            bad.append(("get_dma", nbytes))
        sh.barrier_all()
        torch.cuda.synchronize()
        sh.free(srcsym.data_ptr())
        sh.free(dst.data_ptr())
    if sh.take_status() != 0:
        bad.append(("status",))
    if sh.dma_engines() < 1:
        bad.append(("engines", sh.dma_engines()))
    comm.host_barrier()
    flags = comm.host_all_gather(bytes([1 if bad else 0]))
    if bad:
        print(f"[rank {rank}] SHMEM DMA FAILURES: {bad}", flush=True)
    elif rank == 0:
        print(f"shmem_dma_worker OK on {n} PEs", flush=True)
    sh.finalize()
    comm.destroy()
    sys.exit(1 if any(f[0] for f in flags) else 0)


if __name__ == "__main__":
    main()
