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

#ifdef __cplusplus
}
#endif

#endif /* B200COLL_FUSED_H_ */
