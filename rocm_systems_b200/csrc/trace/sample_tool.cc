// A minimal profiling tool for the b200coll dispatch table: counts calls and bytes per API slot
// and prints a summary at exit. Load it with B200COLL_TOOL_LIBRARIES=/path/libb200coll_sample_tool.so.
// It shows the contract of api_trace.h: save the original slot, install a wrapper, call through
// (the pattern the reference's RCCL wrapper follows, rocprofiler-sdk/source/lib/rocprofiler-sdk/rccl/rccl.cpp:145-265).
#include <stdio.h>
#include <stdlib.h>

#include <atomic>

#include "b200coll/api_trace.h"

namespace {

b200collApiFuncTable gOrig;
std::atomic<unsigned long long> gCalls[B200COLL_API_ID_LAST];
std::atomic<unsigned long long> gBytes{0};

size_t typeBytes(ncclDataType_t t) {
  switch (t) {
    case ncclInt8: case ncclUint8: case ncclFp8E4M3: case ncclFp8E5M2: return 1;
    case ncclFloat16: case ncclBfloat16: return 2;
    case ncclInt32: case ncclUint32: case ncclFloat32: return 4;
    default: return 8;
  }
}

ncclResult_t wrapAllReduce(const void* s, void* r, size_t c, ncclDataType_t dt, ncclRedOp_t op, ncclComm_t comm, cudaStream_t st) {
  gCalls[B200COLL_API_ID_ncclAllReduce]++;
  gBytes += c * typeBytes(dt);
  return gOrig.ncclAllReduce_fn(s, r, c, dt, op, comm, st);
}
ncclResult_t wrapAllGather(const void* s, void* r, size_t c, ncclDataType_t dt, ncclComm_t comm, cudaStream_t st) {
  gCalls[B200COLL_API_ID_ncclAllGather]++;
  gBytes += c * typeBytes(dt);
  return gOrig.ncclAllGather_fn(s, r, c, dt, comm, st);
}
ncclResult_t wrapReduceScatter(const void* s, void* r, size_t c, ncclDataType_t dt, ncclRedOp_t op, ncclComm_t comm, cudaStream_t st) {
  gCalls[B200COLL_API_ID_ncclReduceScatter]++;
  gBytes += c * typeBytes(dt);
  return gOrig.ncclReduceScatter_fn(s, r, c, dt, op, comm, st);
}
ncclResult_t wrapGetVersion(int* v) {
  gCalls[B200COLL_API_ID_ncclGetVersion]++;
  return gOrig.ncclGetVersion_fn(v);
}

void report() {
  const char* out = getenv("B200COLL_SAMPLE_TOOL_OUTPUT");
  FILE* f = out ? fopen(out, "w") : stderr;
  if (!f) return;
  for (int i = 0; i < B200COLL_API_ID_LAST; i++)
    if (gCalls[i].load()) fprintf(f, "%s calls=%llu\n", b200collApiName(i), gCalls[i].load());
  fprintf(f, "payload_bytes=%llu\n", gBytes.load());
  if (out) fclose(f);
}

}  // namespace

extern "C" int b200coll_tool_configure(uint32_t version, b200collApiFuncTable* table, uint64_t libraryId) {
  (void)version;
  (void)libraryId;
  if (!table || table->size < sizeof(b200collApiFuncTable)) return 1;  // older library: slots we need may be missing
  gOrig = *table;
  table->ncclAllReduce_fn = wrapAllReduce;
  table->ncclAllGather_fn = wrapAllGather;
  table->ncclReduceScatter_fn = wrapReduceScatter;
  table->ncclGetVersion_fn = wrapGetVersion;
  atexit(report);
  return 0;
}
