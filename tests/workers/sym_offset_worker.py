"""One rank of the zero-copy agreement check: every rank passes a buffer inside the same symmetric window, but at an offset
that depends on its rank. The zero-copy path would apply each rank's own offset to its peers' mappings and read the wrong
bytes; with B200COLL_CHECK_SYMMETRIC=1 the ranks compare (window, offset) first, find the difference, and all of them
stage. Results are small integers, compared exactly. A second pass at equal offsets must keep the zero-copy path."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402

from rocm_systems_b200.comm import init_from_env  # noqa: E402


def main():
    comm = init_from_env()
    rank, n = comm.rank, comm.nranks
    cnt = 1 << 20
    sym = comm.sym_alloc(4 * cnt * 4)
    bad = []
    for skew in (256, 0):                                      # bytes of offset per rank; 0: the symmetric contract holds
        off = rank * skew
        s_t = sym.tensor((cnt,), torch.float32, offset_bytes=off)
        r_t = sym.tensor((cnt,), torch.float32, offset_bytes=2 * cnt * 4 + off)
        g = torch.Generator().manual_seed(7)
        base = torch.randint(-4, 5, (cnt,), generator=g).float()
        s_t.copy_(base * (rank + 1))
        comm.host_barrier()
        comm.all_reduce(s_t, r_t)
        torch.cuda.synchronize()
        want = (base * (n * (n + 1) // 2)).to(r_t.device)
        if not torch.equal(r_t, want):
            bad.append(("all_reduce", skew, int((r_t != want).sum())))
        per = cnt // n
        out = torch.zeros(per * n, device=r_t.device)
        comm.all_gather(s_t[:per], out)
        torch.cuda.synchronize()
        want_g = torch.cat([base[:per] * (r + 1) for r in range(n)]).to(out.device)
        if not torch.equal(out, want_g):
            bad.append(("all_gather", skew, int((out != want_g).sum())))
        comm.host_barrier()
    err = comm.async_error()
    if err:
        bad.append(("async_error", err, comm.last_error()))
    flags = comm.host_all_gather(bytes([1 if bad else 0]))
    if bad:
        print(f"[rank {rank}] SYMMETRIC OFFSET MISMATCH: {bad}", flush=True)
    elif rank == 0:
        print(f"sym_offset_worker OK on {n} ranks", flush=True)
    torch.cuda.synchronize()
    sym.free()
    comm.destroy()
    sys.exit(1 if any(f[0] for f in flags) else 0)


if __name__ == "__main__":
    main()
