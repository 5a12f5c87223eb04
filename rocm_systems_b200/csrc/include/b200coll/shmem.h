/*
 * b200shmem — OpenSHMEM-style symmetric heap and device-initiated communication on top of a
 * b200coll communicator. Host API in this header; the device API (put/get, signals, atomics,
 * barrier, callable from inside any CUDA kernel) is in b200coll/shmem_device.cuh.
 *
 * The reference snapshot holds no rocSHMEM source; what it has are the primitives such a layer
 * stands on: peer-mapped IPC memory (rocr-runtime/runtime/hsa-runtime/core/runtime/runtime.cpp:1199-1545),
 * cross-process signals (core/runtime/ipc_signal.cpp:71-91) and 64-bit signal atomics with four
 * memory orders (core/runtime/default_signal.cpp:57-250). Here the heap is one symmetric VMM
 * allocation mapped by every PE (plus its NVSwitch multicast alias), signals are 64-bit words in
 * that heap, and every wait carries a time budget after which it returns a status instead of
 * spinning on.
 */
#ifndef B200COLL_SHMEM_H_
#define B200COLL_SHMEM_H_

#include "b200coll/nccl.h"

#ifdef __cplusplus
extern "C" {
#endif

#define B200SHMEM_MAX_PES 8
#define B200SHMEM_MAX_DMA_GANG 8

/* What a kernel needs to talk to its peers; passed by value as a kernel argument. */
typedef struct b200shmem_dev {
  int pe, npes;
  char* heap[B200SHMEM_MAX_PES];  /* this PE's mapping of every PE's heap; heap[pe] is local */
  char* heapMc;                   /* multicast alias of the heap (multimem.* only), or NULL */
  unsigned long long heapBytes;
  unsigned long long* syncFlags;  /* local: [B200SHMEM_MAX_PES] arrival words of barrier_all, inside the heap */
  unsigned long long* syncEpoch;  /* local device memory: barriers completed so far */
  int* status;                    /* local device memory: first failed wait (0 none) */
  unsigned long long timeoutNs;   /* budget of every device-side wait */
} b200shmem_dev_t;

/* A team: the PEs start, start + stride, ..., size of them (OpenSHMEM teams). Passed by value to kernels next to the
 * device context. Its barrier words are a slot of their own in the heap's reserved head, so teams synchronise
 * independently of one another and of barrier_all. */
typedef struct b200shmem_team {
  int start, stride, size;
  int idx;                        /* this PE's index in the team, or -1 when it is not a member */
  unsigned long long* syncFlags;  /* local: [B200SHMEM_MAX_PES] arrival words of this team, indexed by team index */
  unsigned long long* syncEpoch;  /* local device memory: barriers of this team completed so far */
} b200shmem_team_t;
#define B200SHMEM_MAX_TEAMS 64

typedef struct b200shmem_ctx* b200shmem_ctx_t;

enum { B200SHMEM_CMP_EQ = 0, B200SHMEM_CMP_NE, B200SHMEM_CMP_GT, B200SHMEM_CMP_GE, B200SHMEM_CMP_LT, B200SHMEM_CMP_LE };
enum { B200SHMEM_SIGNAL_SET = 0, B200SHMEM_SIGNAL_ADD = 1 };
enum { B200SHMEM_OK = 0, B200SHMEM_TIMEOUT = 1 };

/* Collective over `comm`: reserve a symmetric heap of `heapBytes` on every PE. */
ncclResult_t b200shmem_init(ncclComm_t comm, size_t heapBytes, b200shmem_ctx_t* ctx);
ncclResult_t b200shmem_finalize(b200shmem_ctx_t ctx);
int b200shmem_my_pe(b200shmem_ctx_t ctx);
int b200shmem_n_pes(b200shmem_ctx_t ctx);
/* Symmetric allocation: every PE must make the same sequence of malloc/free calls, which is what
 * makes offsets agree (the OpenSHMEM rule). Returns NULL when the heap is exhausted. */
void* b200shmem_malloc(b200shmem_ctx_t ctx, size_t size);
void* b200shmem_align(b200shmem_ctx_t ctx, size_t alignment, size_t size);
void b200shmem_free(b200shmem_ctx_t ctx, void* ptr);
/* Address through which this PE reaches `pe`'s copy of a symmetric object. */
void* b200shmem_ptr(b200shmem_ctx_t ctx, const void* ptr, int pe);
void* b200shmem_mc_ptr(b200shmem_ctx_t ctx, const void* ptr);
ncclResult_t b200shmem_device_ctx(b200shmem_ctx_t ctx, b200shmem_dev_t* out);
/* Teams. team_world gives the team of all PEs (it shares barrier_all's words). team_split_strided makes the team of the
 * parent's members start, start + stride, ... (`size` of them, indices in the PARENT team); it must be called by EVERY PE
 * of the context in the same order, members or not (that is what keeps the teams' barrier slots in step); a PE that is
 * not a member gets idx == -1 and must not use the team in a collective. At most B200SHMEM_MAX_TEAMS - 1 splits per
 * context; team_destroy releases nothing that could be reused and exists for symmetry. */
ncclResult_t b200shmem_team_world(b200shmem_ctx_t ctx, b200shmem_team_t* team);
ncclResult_t b200shmem_team_split_strided(b200shmem_ctx_t ctx, const b200shmem_team_t* parent, int start, int stride, int size, b200shmem_team_t* team);
void b200shmem_team_destroy(b200shmem_ctx_t ctx, b200shmem_team_t* team);
int b200shmem_team_my_pe(const b200shmem_team_t* team);
int b200shmem_team_n_pes(const b200shmem_team_t* team);
/* PE number in `dst` of member `idx` of `src`, or -1 when it is not a member of `dst`. */
int b200shmem_team_translate_pe(const b200shmem_team_t* src, int idx, const b200shmem_team_t* dst);
ncclResult_t b200shmem_team_sync_on_stream(b200shmem_ctx_t ctx, const b200shmem_team_t* team, cudaStream_t stream);
/* Stream-ordered host-initiated operations. */
ncclResult_t b200shmem_putmem_on_stream(b200shmem_ctx_t ctx, void* dest, const void* source, size_t bytes, int pe, cudaStream_t stream);
ncclResult_t b200shmem_getmem_on_stream(b200shmem_ctx_t ctx, void* dest, const void* source, size_t bytes, int pe, cudaStream_t stream);
ncclResult_t b200shmem_putmem_signal_on_stream(b200shmem_ctx_t ctx, void* dest, const void* source, size_t bytes, unsigned long long* sigAddr,
                                               unsigned long long signal, int sigOp, int pe, cudaStream_t stream);
ncclResult_t b200shmem_signal_wait_until_on_stream(b200shmem_ctx_t ctx, unsigned long long* sigAddr, int cmp, unsigned long long value,
                                                   cudaStream_t stream);
ncclResult_t b200shmem_barrier_all_on_stream(b200shmem_ctx_t ctx, cudaStream_t stream);
/* Copy-engine variants of put / get / put+signal: the bytes move by DMA, no SM takes part, and a large transfer is
 * split over `gang` engines (0: chosen from the size, or B200COLL_DMA_GANG). They are stream-ordered like the others
 * and can be captured into a CUDA graph. The signal of the put+signal form is stored by one warp after the copies. */
ncclResult_t b200shmem_putmem_dma_on_stream(b200shmem_ctx_t ctx, void* dest, const void* source, size_t bytes, int pe, int gang, cudaStream_t stream);
ncclResult_t b200shmem_getmem_dma_on_stream(b200shmem_ctx_t ctx, void* dest, const void* source, size_t bytes, int pe, int gang, cudaStream_t stream);
ncclResult_t b200shmem_putmem_signal_dma_on_stream(b200shmem_ctx_t ctx, void* dest, const void* source, size_t bytes, unsigned long long* sigAddr,
                                                   unsigned long long signal, int sigOp, int pe, int gang, cudaStream_t stream);
/* How a transfer of `bytes` is cut: returns the number of parts and fills offsets/lengths (each may be NULL). Pure. */
int b200shmem_dma_plan(size_t bytes, int gang, size_t* offsets, size_t* lengths);
/* Number of asynchronous copy engines of this PE's GPU, or -1. */
int b200shmem_dma_engines(b200shmem_ctx_t ctx);
/* First device-side wait that ran out of budget since the last call (B200SHMEM_OK if none); synchronises the device. */
int b200shmem_take_status(b200shmem_ctx_t ctx);

/* Self-checks that run device-initiated traffic from inside kernels (used by the tests):
 * ring: every PE puts `count` words to its right neighbour with put+signal, waits for its own
 * signal, and verifies; atomics: every PE does fetch-add/compare-swap/and/or/xor/swap rounds on
 * PE 0's words. Return the number of mismatches in *errors. */
ncclResult_t b200shmem_selftest_ring(b200shmem_ctx_t ctx, size_t count, int rounds, cudaStream_t stream, int* errors);
ncclResult_t b200shmem_selftest_atomics(b200shmem_ctx_t ctx, int iters, cudaStream_t stream, int* errors);
/* The device API's block-scope collectives (broadcast, fcollect, alltoall, sum / max reduce), wait_until / test and the
 * strided put on `count` 64-bit words per block, each checked against its closed form. Collective over the PEs. */
ncclResult_t b200shmem_selftest_collectives(b200shmem_ctx_t ctx, size_t count, cudaStream_t stream, int* errors);
/* The same collectives inside teams: the PEs are split into the even and the odd ones (and, from four PEs up, the even
 * team once more), every team runs sync / broadcast / fcollect / alltoall / sum reduce on its own members at the same
 * time as the others. Collective over all PEs. */
ncclResult_t b200shmem_selftest_teams(b200shmem_ctx_t ctx, size_t count, cudaStream_t stream, int* errors);

/* The two self-checks between `n` PEs that share the current GPU (communicators created under B200COLL_EMULATE_RANKS=1):
 * every PE is one block of a single cooperative kernel. For tests on one GPU. */
ncclResult_t b200shmem_emu_selftest(ncclComm_t* comms, int n, size_t count, int rounds, int iters, int* errors);

#ifdef __cplusplus
}
#endif

#endif /* B200COLL_SHMEM_H_ */
