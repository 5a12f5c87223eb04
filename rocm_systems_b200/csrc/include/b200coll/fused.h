/*
 * Fused compute + communication entry points of b200coll (no counterpart in the NCCL API).
 * All of them enqueue on `stream` and return at once; buffers are device pointers.
 */
#ifndef B200COLL_FUSED_H_
#define B200COLL_FUSED_H_

#include "b200coll/nccl.h"

#ifdef __cplusplus
extern "C" {
#endif

/* FSDP gradient bucket: reduce-scatter of bf16 inputs (nranks * recvcount elements per rank)
 * with fp32 accumulation, multiplied by `scale`, written as fp32 (recvcount elements). */
ncclResult_t b200collReduceScatterCast(ncclComm_t comm, const void* sendBf16, float* recvF32, size_t recvcount, float scale,
                                       cudaStream_t stream);

/* Tensor-parallel all-gather -> GEMM in one tcgen05 kernel.
 * xSym: this rank's copy of X [nranks * rowsPerRank, K] bf16 inside symmetric memory, with this
 * rank's shard already at rows [rank * rowsPerRank, +rowsPerRank). The kernel pulls the other
 * shards from the peers while it multiplies: out = X * w^T with w [wRows, K] bf16 (K-major).
 * swiglu != 0: w holds, per block of 256 (or 128) rows, first the gate rows then the up rows of
 * the same outputs, and out [M, wRows / 2] = silu(gate) * up; else out is [M, wRows].
 * commCtas: CTAs that move data (0 = default). */
ncclResult_t b200collAgGemm(ncclComm_t comm, void* xSym, const void* w, void* out, int rowsPerRank, int wRows, int K, int swiglu,
                            int commCtas, cudaStream_t stream);

/* Tensor-parallel GEMM -> reduce-scatter in one tcgen05 kernel.
 * a [nranks * rowsPerRank, K] bf16 and w [N, K] bf16 are this rank's K-shards; y [rowsPerRank, N]
 * bf16 receives rows [rank * rowsPerRank, +rowsPerRank) of sum_over_ranks(a * w^T).
 * workspaceSym: zero-initialised symmetric memory of b200collGemmRsWorkspaceBytes() bytes, the
 * same allocation on every call of a sequence. */
size_t b200collGemmRsWorkspaceBytes(int rowsPerRank, int N, int nranks);
ncclResult_t b200collGemmRs(ncclComm_t comm, const void* a, const void* w, void* workspaceSym, void* y, int rowsPerRank, int N, int K,
                            cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* B200COLL_FUSED_H_ */
