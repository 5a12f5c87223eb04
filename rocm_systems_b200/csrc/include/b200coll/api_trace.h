/*
 * Interceptable dispatch table of the b200coll public API.
 *
 * Same idea and slot order as the 37-entry rcclApiFuncTable that RCCL hands to profilers
 * (rocprofiler-sdk/source/include/rocprofiler-sdk/rccl/details/api_trace.h:204-243; slot ids
 * rocprofiler-sdk/source/include/rocprofiler-sdk/rccl/api_id.h:32-72). Every un-prefixed public
 * entry point calls through this table. A tool named in B200COLL_TOOL_LIBRARIES (or linked into
 * the process) that exports
 *     int b200coll_tool_configure(uint32_t version, b200collApiFuncTable* table, uint64_t id);
 * receives the table once, before the first call goes through it, and may save and replace any
 * slot. The layout is ABI: `size` first, then one pointer per slot, in this order, forever;
 * new slots are appended.
 */
#ifndef B200COLL_API_TRACE_H_
#define B200COLL_API_TRACE_H_

#include "b200coll/nccl.h"

#ifdef __cplusplus
extern "C" {
#endif

#define B200COLL_API_TRACE_VERSION_MAJOR 0
#define B200COLL_API_TRACE_VERSION_PATCH 1

typedef enum {
  B200COLL_API_ID_NONE = -1,
  B200COLL_API_ID_ncclAllGather = 0,
  B200COLL_API_ID_ncclAllReduce,
  B200COLL_API_ID_ncclAllToAll,
  B200COLL_API_ID_ncclAllToAllv,
  B200COLL_API_ID_ncclBroadcast,
  B200COLL_API_ID_ncclGather,
  B200COLL_API_ID_ncclReduce,
  B200COLL_API_ID_ncclReduceScatter,
  B200COLL_API_ID_ncclScatter,
  B200COLL_API_ID_ncclSend,
  B200COLL_API_ID_ncclRecv,
  B200COLL_API_ID_ncclRedOpCreatePreMulSum,
  B200COLL_API_ID_ncclRedOpDestroy,
  B200COLL_API_ID_ncclGroupStart,
  B200COLL_API_ID_ncclGroupEnd,
  B200COLL_API_ID_ncclGetVersion,
  B200COLL_API_ID_ncclGetUniqueId,
  B200COLL_API_ID_ncclCommInitRank,
  B200COLL_API_ID_ncclCommInitAll,
  B200COLL_API_ID_ncclCommInitRankConfig,
  B200COLL_API_ID_ncclCommFinalize,
  B200COLL_API_ID_ncclCommDestroy,
  B200COLL_API_ID_ncclCommAbort,
  B200COLL_API_ID_ncclCommSplit,
  B200COLL_API_ID_ncclGetErrorString,
  B200COLL_API_ID_ncclGetLastError,
  B200COLL_API_ID_ncclCommGetAsyncError,
  B200COLL_API_ID_ncclCommCount,
  B200COLL_API_ID_ncclCommCuDevice,
  B200COLL_API_ID_ncclCommUserRank,
  B200COLL_API_ID_ncclMemAlloc,
  B200COLL_API_ID_ncclMemFree,
  B200COLL_API_ID_mscclLoadAlgo,
  B200COLL_API_ID_mscclRunAlgo,
  B200COLL_API_ID_mscclUnloadAlgo,
  B200COLL_API_ID_ncclCommRegister,
  B200COLL_API_ID_ncclCommDeregister,
  B200COLL_API_ID_LAST
} b200collApiId;

typedef struct b200collApiFuncTable {
  uint64_t size;
  ncclResult_t (*ncclAllGather_fn)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*ncclAllReduce_fn)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*ncclAllToAll_fn)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*ncclAllToAllv_fn)(const void*, const size_t[], const size_t[], void*, const size_t[], const size_t[], ncclDataType_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*ncclBroadcast_fn)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*ncclGather_fn)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*ncclReduce_fn)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*ncclReduceScatter_fn)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*ncclScatter_fn)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*ncclSend_fn)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*ncclRecv_fn)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*ncclRedOpCreatePreMulSum_fn)(ncclRedOp_t*, void*, ncclDataType_t, ncclScalarResidence_t, ncclComm_t);
  ncclResult_t (*ncclRedOpDestroy_fn)(ncclRedOp_t, ncclComm_t);
  ncclResult_t (*ncclGroupStart_fn)(void);
  ncclResult_t (*ncclGroupEnd_fn)(void);
  ncclResult_t (*ncclGetVersion_fn)(int*);
  ncclResult_t (*ncclGetUniqueId_fn)(ncclUniqueId*);
  ncclResult_t (*ncclCommInitRank_fn)(ncclComm_t*, int, ncclUniqueId, int);
  ncclResult_t (*ncclCommInitAll_fn)(ncclComm_t*, int, const int*);
  ncclResult_t (*ncclCommInitRankConfig_fn)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*);
  ncclResult_t (*ncclCommFinalize_fn)(ncclComm_t);
  ncclResult_t (*ncclCommDestroy_fn)(ncclComm_t);
  ncclResult_t (*ncclCommAbort_fn)(ncclComm_t);
  ncclResult_t (*ncclCommSplit_fn)(ncclComm_t, int, int, ncclComm_t*, ncclConfig_t*);
  const char* (*ncclGetErrorString_fn)(ncclResult_t);
  const char* (*ncclGetLastError_fn)(ncclComm_t);
  ncclResult_t (*ncclCommGetAsyncError_fn)(ncclComm_t, ncclResult_t*);
  ncclResult_t (*ncclCommCount_fn)(const ncclComm_t, int*);
  ncclResult_t (*ncclCommCuDevice_fn)(const ncclComm_t, int*);
  ncclResult_t (*ncclCommUserRank_fn)(const ncclComm_t, int*);
  ncclResult_t (*ncclMemAlloc_fn)(void**, size_t);
  ncclResult_t (*ncclMemFree_fn)(void*);
  ncclResult_t (*mscclLoadAlgo_fn)(const char*, mscclAlgoHandle_t*, int);
  ncclResult_t (*mscclRunAlgo_fn)(const void*, const size_t[], const size_t[], void*, const size_t[], const size_t[], size_t, ncclDataType_t, int, int, ncclRedOp_t, mscclAlgoHandle_t, ncclComm_t, cudaStream_t);
  ncclResult_t (*mscclUnloadAlgo_fn)(mscclAlgoHandle_t);
  ncclResult_t (*ncclCommRegister_fn)(const ncclComm_t, void*, size_t, void**);
  ncclResult_t (*ncclCommDeregister_fn)(const ncclComm_t, void*);
} b200collApiFuncTable;

typedef int (*b200collToolConfigure_fn)(uint32_t version, b200collApiFuncTable* table, uint64_t libraryId);

/* The live table (for tests and in-process tools). */
b200collApiFuncTable* b200collGetApiTable(void);

/* Built-in tracer access (records exist when B200COLL_TRACE=1 or after b200collTraceEnable). */
typedef struct {
  uint64_t correlationId;
  int32_t opId;
  int32_t dtype;
  uint64_t count;
  uint64_t bytes;
  int32_t algo;
  int32_t ctas;
  uint64_t hostBeginNs;
  uint64_t hostEndNs;
  uint64_t devBeginNs;
  uint64_t devEndNs;
} b200collTraceRecordC;
ncclResult_t b200collTraceEnable(ncclComm_t comm, int on);
/* Synchronises the device, then copies up to `max` records; returns how many exist in *n. */
ncclResult_t b200collTraceGet(ncclComm_t comm, b200collTraceRecordC* out, size_t max, size_t* n);
/* Records that were not kept because B200COLL_TRACE_MAX_RECORDS was reached (0 without a limit). */
ncclResult_t b200collTraceDropped(ncclComm_t comm, uint64_t* dropped);
ncclResult_t b200collTraceClear(ncclComm_t comm);
ncclResult_t b200collTraceWrite(ncclComm_t comm, const char* path, const char* format /* "csv" | "perfetto" */);
const char* b200collApiName(int apiId);

#ifdef __cplusplus
}
#endif

#endif /* B200COLL_API_TRACE_H_ */
