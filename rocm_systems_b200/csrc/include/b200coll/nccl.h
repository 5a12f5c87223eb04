/*
 * b200coll — NCCL-compatible public C API of the Blackwell-native collective library.
 *
 * The surface (types, enum values, entry points) follows the NCCL 2.20.5 / RCCL contract
 * recorded in the reference profiler SDK
 * (rocprofiler-sdk/source/include/rocprofiler-sdk/rccl/details/rccl.h:15-1075) so that a
 * program written against that header recompiles against this one with `cudaStream_t`
 * in place of `hipStream_t`. Every entry point also exists with a `p` prefix
 * (`pncclAllReduce` …, rccl.h:655-662): the un-prefixed symbol goes through the
 * interceptable dispatch table (see api_trace.h), the prefixed one calls the
 * implementation directly.
 */
#ifndef B200COLL_NCCL_H_
#define B200COLL_NCCL_H_

#include <cuda_runtime_api.h>
#include <limits.h>
#include <stddef.h>
#include <stdint.h>

#define NCCL_MAJOR 2
#define NCCL_MINOR 20
#define NCCL_PATCH 5
#define NCCL_SUFFIX "+b200coll"
#define NCCL_VERSION_CODE 22005
#define NCCL_VERSION(X, Y, Z) \
  (((X) <= 2 && (Y) <= 8) ? (X) * 1000 + (Y) * 100 + (Z) : (X) * 10000 + (Y) * 100 + (Z))

/* Feature macros a caller can test, mirroring the RCCL_* feature switches. */
#define B200COLL 1
#define RCCL_BFLOAT16 1
#define RCCL_FLOAT8 1
#define RCCL_GATHER_SCATTER 1
#define RCCL_ALLTOALLV 1

#ifdef __cplusplus
extern "C" {
#endif

typedef const struct ncclComm* ncclComm_t;
#define NCCL_COMM_NULL NULL

#define NCCL_UNIQUE_ID_BYTES 128
typedef struct {
  char internal[NCCL_UNIQUE_ID_BYTES];
} ncclUniqueId;

typedef enum {
  ncclSuccess = 0,
  ncclUnhandledCudaError = 1,
  ncclSystemError = 2,
  ncclInternalError = 3,
  ncclInvalidArgument = 4,
  ncclInvalidUsage = 5,
  ncclRemoteError = 6,
  ncclInProgress = 7,
  ncclNumResults = 8
} ncclResult_t;

#define NCCL_CONFIG_UNDEF_INT INT_MIN
#define NCCL_CONFIG_UNDEF_PTR NULL
#define NCCL_SPLIT_NOCOLOR -1

typedef struct ncclConfig_v21700 {
  size_t size;          /* filled by NCCL_CONFIG_INITIALIZER */
  unsigned int magic;   /* filled by NCCL_CONFIG_INITIALIZER */
  unsigned int version; /* filled by NCCL_CONFIG_INITIALIZER */
  int blocking;         /* 1: calls return when enqueued; 0: init/finalize may return ncclInProgress */
  int cgaClusterSize;   /* accepted; kernels here do not use clusters across ranks */
  int minCTAs;          /* lower bound on CTAs per collective kernel */
  int maxCTAs;          /* upper bound on CTAs per collective kernel */
  const char* netName;  /* accepted and ignored: single NVSwitch domain */
  int splitShare;       /* accepted; split communicators get their own workspace */
} ncclConfig_t;

#define NCCL_CONFIG_INITIALIZER                                                               \
  {                                                                                           \
    sizeof(ncclConfig_t), 0xcafebeef, NCCL_VERSION(NCCL_MAJOR, NCCL_MINOR, NCCL_PATCH),       \
        NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT,                  \
        NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_PTR, NCCL_CONFIG_UNDEF_INT                   \
  }

typedef enum { ncclNumOps_dummy = 5 } ncclRedOp_dummy_t;
typedef enum {
  ncclSum = 0,
  ncclProd = 1,
  ncclMax = 2,
  ncclMin = 3,
  ncclAvg = 4,
  ncclNumOps = 5, /* dynamic operators made by ncclRedOpCreate* are >= this */
  ncclMaxRedOp = 0x7fffffff >> (32 - 8 * sizeof(ncclRedOp_dummy_t))
} ncclRedOp_t;

typedef enum {
  ncclInt8 = 0,
  ncclChar = 0,
  ncclUint8 = 1,
  ncclInt32 = 2,
  ncclInt = 2,
  ncclUint32 = 3,
  ncclInt64 = 4,
  ncclUint64 = 5,
  ncclFloat16 = 6,
  ncclHalf = 6,
  ncclFloat32 = 7,
  ncclFloat = 7,
  ncclFloat64 = 8,
  ncclDouble = 8,
  ncclBfloat16 = 9,
  ncclFp8E4M3 = 10, /* OCP e4m3 (finite, NaN = 0x7f/0xff) as used by Blackwell tensor cores */
  ncclFp8E5M2 = 11, /* OCP e5m2 */
  ncclNumTypes = 12
} ncclDataType_t;

typedef enum { ncclScalarDevice = 0, ncclScalarHostImmediate = 1 } ncclScalarResidence_t;

typedef int mscclAlgoHandle_t;

#define B200COLL_DECL(ret, name, ...) \
  ret name(__VA_ARGS__);              \
  ret p##name(__VA_ARGS__);

/* Memory that can be mapped into every rank of a communicator (CUDA VMM allocation with a
 * shareable handle). Buffers from here, once registered, take the zero-copy paths. */
B200COLL_DECL(ncclResult_t, ncclMemAlloc, void** ptr, size_t size)
B200COLL_DECL(ncclResult_t, ncclMemFree, void* ptr)

B200COLL_DECL(ncclResult_t, ncclGetVersion, int* version)
B200COLL_DECL(ncclResult_t, ncclGetUniqueId, ncclUniqueId* uniqueId)
B200COLL_DECL(ncclResult_t, ncclCommInitRankConfig, ncclComm_t* comm, int nranks,
              ncclUniqueId commId, int rank, ncclConfig_t* config)
B200COLL_DECL(ncclResult_t, ncclCommInitRank, ncclComm_t* comm, int nranks, ncclUniqueId commId,
              int rank)
B200COLL_DECL(ncclResult_t, ncclCommInitAll, ncclComm_t* comm, int ndev, const int* devlist)
B200COLL_DECL(ncclResult_t, ncclCommFinalize, ncclComm_t comm)
B200COLL_DECL(ncclResult_t, ncclCommDestroy, ncclComm_t comm)
B200COLL_DECL(ncclResult_t, ncclCommAbort, ncclComm_t comm)
B200COLL_DECL(ncclResult_t, ncclCommSplit, ncclComm_t comm, int color, int key,
              ncclComm_t* newcomm, ncclConfig_t* config)
B200COLL_DECL(const char*, ncclGetErrorString, ncclResult_t result)
B200COLL_DECL(const char*, ncclGetLastError, ncclComm_t comm)
B200COLL_DECL(ncclResult_t, ncclCommGetAsyncError, ncclComm_t comm, ncclResult_t* asyncError)
B200COLL_DECL(ncclResult_t, ncclCommCount, const ncclComm_t comm, int* count)
B200COLL_DECL(ncclResult_t, ncclCommCuDevice, const ncclComm_t comm, int* device)
B200COLL_DECL(ncclResult_t, ncclCommUserRank, const ncclComm_t comm, int* rank)
/* Registration is local and cheap; the peer mapping of a registered buffer is exchanged the
 * first time a collective uses it, so every rank must register the matching buffer. */
B200COLL_DECL(ncclResult_t, ncclCommRegister, const ncclComm_t comm, void* buff, size_t size,
              void** handle)
B200COLL_DECL(ncclResult_t, ncclCommDeregister, const ncclComm_t comm, void* handle)

B200COLL_DECL(ncclResult_t, ncclRedOpCreatePreMulSum, ncclRedOp_t* op, void* scalar,
              ncclDataType_t datatype, ncclScalarResidence_t residence, ncclComm_t comm)
B200COLL_DECL(ncclResult_t, ncclRedOpDestroy, ncclRedOp_t op, ncclComm_t comm)

B200COLL_DECL(ncclResult_t, ncclReduce, const void* sendbuff, void* recvbuff, size_t count,
              ncclDataType_t datatype, ncclRedOp_t op, int root, ncclComm_t comm,
              cudaStream_t stream)
B200COLL_DECL(ncclResult_t, ncclBcast, void* buff, size_t count, ncclDataType_t datatype, int root,
              ncclComm_t comm, cudaStream_t stream)
B200COLL_DECL(ncclResult_t, ncclBroadcast, const void* sendbuff, void* recvbuff, size_t count,
              ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream)
B200COLL_DECL(ncclResult_t, ncclAllReduce, const void* sendbuff, void* recvbuff, size_t count,
              ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream)
/* In place when recvbuff == sendbuff + rank * recvcount (rccl.h:665-671). */
B200COLL_DECL(ncclResult_t, ncclReduceScatter, const void* sendbuff, void* recvbuff,
              size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm,
              cudaStream_t stream)
/* In place when sendbuff == recvbuff + rank * sendcount (rccl.h:700-705). */
B200COLL_DECL(ncclResult_t, ncclAllGather, const void* sendbuff, void* recvbuff, size_t sendcount,
              ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream)
/* Send/Recv to make progress together must sit in one group (rccl.h:731-737). */
B200COLL_DECL(ncclResult_t, ncclSend, const void* sendbuff, size_t count, ncclDataType_t datatype,
              int peer, ncclComm_t comm, cudaStream_t stream)
B200COLL_DECL(ncclResult_t, ncclRecv, void* recvbuff, size_t count, ncclDataType_t datatype,
              int peer, ncclComm_t comm, cudaStream_t stream)
B200COLL_DECL(ncclResult_t, ncclGather, const void* sendbuff, void* recvbuff, size_t sendcount,
              ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream)
B200COLL_DECL(ncclResult_t, ncclScatter, const void* sendbuff, void* recvbuff, size_t recvcount,
              ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream)
/* Not in place (rccl.h:864-869). */
B200COLL_DECL(ncclResult_t, ncclAllToAll, const void* sendbuff, void* recvbuff, size_t count,
              ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream)
B200COLL_DECL(ncclResult_t, ncclAllToAllv, const void* sendbuff, const size_t sendcounts[],
              const size_t sdispls[], void* recvbuff, const size_t recvcounts[],
              const size_t rdispls[], ncclDataType_t datatype, ncclComm_t comm,
              cudaStream_t stream)

/* Schedule files: a small JSON document naming a collective and forcing algorithm / CTA
 * choices for it (the role MSCCL algorithm files play in rccl.h:955-1030). */
B200COLL_DECL(ncclResult_t, mscclLoadAlgo, const char* mscclAlgoFilePath,
              mscclAlgoHandle_t* mscclAlgoHandle, int rank)
B200COLL_DECL(ncclResult_t, mscclRunAlgo, const void* sendBuff, const size_t sendCounts[],
              const size_t sDisPls[], void* recvBuff, const size_t recvCounts[],
              const size_t rDisPls[], size_t count, ncclDataType_t dataType, int root, int peer,
              ncclRedOp_t op, mscclAlgoHandle_t mscclAlgoHandle, ncclComm_t comm,
              cudaStream_t stream)
B200COLL_DECL(ncclResult_t, mscclUnloadAlgo, mscclAlgoHandle_t mscclAlgoHandle)

B200COLL_DECL(ncclResult_t, ncclGroupStart, void)
B200COLL_DECL(ncclResult_t, ncclGroupEnd, void)

#undef B200COLL_DECL

/* ---- Extensions (no counterpart in NCCL 2.20): symmetric windows ------------------------ */

/* Collective: every rank of `comm` allocates `size` bytes that all ranks map. `*ptr` is the
 * local address; collectives whose buffers lie in such a window skip the staging copies.
 *
 * The symmetric contract. A collective takes that zero-copy path when, on the calling rank, its
 * buffers lie inside windows (these, or ncclMemAlloc memory after ncclCommRegister) and are 16-byte
 * aligned; it then reaches every peer's buffer at the SAME offset of the SAME window. So all ranks
 * of one call must pass the same place: window created by the same collective call, equal offset,
 * or all of them ordinary memory. A call that mixes them computes on the wrong bytes or runs into
 * its wait limit. With B200COLL_CHECK_SYMMETRIC=1 the ranks compare window and offset over the
 * rendezvous network before each collective and all stage when they differ (one host exchange per
 * call: a debugging aid). Windows must be created in the same order on every rank. */
ncclResult_t b200collSymAlloc(ncclComm_t comm, size_t size, void** ptr);
ncclResult_t b200collSymFree(ncclComm_t comm, void* ptr);
/* Address through which this rank reaches `peer`'s copy of a symmetric pointer. */
ncclResult_t b200collSymPeerPtr(ncclComm_t comm, const void* ptr, int peer, void** peerPtr);
/* Multicast (NVLS) alias of a symmetric pointer, or NULL when the box has no multicast. */
ncclResult_t b200collSymMulticastPtr(ncclComm_t comm, const void* ptr, void** mcPtr);
/* Host-side barrier over the bootstrap network (no GPU work). */
ncclResult_t b200collHostBarrier(ncclComm_t comm);
/* All-gather `bytes` bytes per rank over the bootstrap network (host memory). */
ncclResult_t b200collHostAllGather(ncclComm_t comm, const void* send, void* recv, size_t bytes);
/* Device-side barrier enqueued on `stream`. */
ncclResult_t b200collBarrier(ncclComm_t comm, cudaStream_t stream);

/* ---- Extensions for tests on a single GPU: several ranks played by one cooperative kernel --------
 * With B200COLL_EMULATE_RANKS=1 (and B200COLL_NVLS_ENABLE=0) ncclCommInitAll accepts the same device several times.
 * Such communicators refuse every launching entry point except these: separate kernels of ranks that wait on one
 * another must never share a GPU. kind: 0 all-reduce, 1 reduce-scatter, 2 reduce, 3 all-gather, 4 broadcast; types
 * float, bfloat16, int32; operators sum, max, avg. send[r] / recv[r] are rank r's buffers. */
ncclResult_t b200collEmuCollective(ncclComm_t* comms, int n, int kind, const void* const* send, void* const* recv, size_t count, ncclDataType_t dt,
                                   ncclRedOp_t op, int root, int ctasPerRank, cudaStream_t stream);
/* All-to-all of bytesPerPeer bytes per pair through the grouped send/recv kernel (FIFO slots and credits). */
ncclResult_t b200collEmuAllToAll(ncclComm_t* comms, int n, const void* const* send, void* const* recv, size_t bytesPerPeer, cudaStream_t stream);
/* The fused gradient reduce-scatter of the FSDP path on such communicators: send[r] holds n * recvcount bf16 values,
 * recv[r] receives rank r's recvcount fp32 sums times `scale`. */
ncclResult_t b200collEmuReduceScatterCast(ncclComm_t* comms, int n, const void* const* send, float* const* recv, size_t recvcount, float scale,
                                          int ctasPerRank, cudaStream_t stream);
/* Creates `nranks` such communicators on the current GPU, runs every collective in the three types and the fused
 * reduce-scatter on `count` elements, verifies on the host; *wrong = wrong elements, *status = first asynchronous error of any rank. */
ncclResult_t b200collEmuSelftest(int nranks, size_t count, long long* wrong, int* status);

/* ---- Extensions that need no GPU: what the planner would do, and the settings ------------ */

/* What the planner chooses for a collective on a communicator of `nranks` ranks, with or without a multicast
 * alias: algo 1 flag-in-data, 2 peer loads, 3 in-switch; CTAs; zero-copy (never here: the buffers are in no window);
 * pipeline chunks. Honours the environment and the tuning file exactly as a real communicator does.
 * kind: 0 all-reduce, 1 reduce-scatter, 2 reduce, 3 all-gather, 4 broadcast. */
typedef struct b200collPlanInfo {
  int algo, ctas, direct;
  unsigned long long chunks;
} b200collPlanInfo;
ncclResult_t b200collPlanDry(int nranks, int nvls, int kind, size_t count, ncclDataType_t dt, ncclRedOp_t op, b200collPlanInfo* out);
/* JSON description of every setting (environment names, current value, default, meaning) copied into `buf`
 * (NUL-terminated, truncated to `cap`); returns the size the whole text needs. */
size_t b200collDescribeSettings(char* buf, size_t cap);

#ifdef __cplusplus
}
#endif

#endif /* B200COLL_NCCL_H_ */
