/*
 * b200prof — activity tracing for any CUDA program on the device: kernel dispatches, memory
 * copies / sets and CUDA API calls with one clock (CLOCK_MONOTONIC) shared with the collective
 * tracer and the b200tx markers. It plays the part of the reference's profiling SDK and its
 * tool library (rocprofiler-sdk/source/include/rocprofiler-sdk/{buffer_tracing,callback_tracing}.h,
 * rocprofiler-sdk/source/lib/rocprofiler-sdk-tool/tool.cpp) on top of CUPTI's activity API.
 *
 * Two ways in:
 *   - in process: b200profStart(kinds) ... b200profStop(), then read or write the records;
 *   - from outside: CUDA_INJECTION64_PATH=<libb200prof.so> makes the CUDA driver load the library
 *     and call InitializeInjection(); the B200PROF_* variables choose what is traced and where the
 *     CSV files go (the tracing launcher `tools/prof.py` sets them).
 */
#ifndef B200COLL_PROF_H_
#define B200COLL_PROF_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  B200PROF_KERNEL = 1,       /* kernel dispatches */
  B200PROF_MEMOP = 2,        /* memcpy (incl. peer to peer) and memset */
  B200PROF_RUNTIME_API = 4,  /* cuda* calls */
  B200PROF_DRIVER_API = 8,   /* cu* calls */
  B200PROF_SYNC = 16         /* stream / event / context synchronisation */
};

typedef struct {
  uint64_t startNs, endNs;
  uint32_t device, context, stream, correlationId;
  int32_t grid[3], block[3];
  uint32_t cluster[3];
  int32_t staticSmem, dynamicSmem;
  uint32_t registersPerThread, localPerThread;
  uint64_t graphNodeId;
  char name[192]; /* demangled, truncated */
} b200prof_kernel_t;

typedef struct {
  uint64_t startNs, endNs, bytes;
  uint32_t device, context, stream, correlationId;
  uint8_t op;      /* 0 memcpy, 1 peer-to-peer memcpy, 2 memset */
  uint8_t copyKind, srcKind, dstKind; /* CUPTI's CUpti_ActivityMemcpyKind / MemoryKind values */
  uint32_t srcDevice, dstDevice;      /* peer-to-peer copies only */
} b200prof_memop_t;

typedef struct {
  uint64_t startNs, endNs;
  uint32_t cbid, processId, threadId, correlationId, returnValue;
  uint32_t domain; /* 0 runtime, 1 driver, 2 synchronisation */
  char name[64];
} b200prof_api_t;

int b200profStart(unsigned kinds);   /* 0 on success; a second Start while running adds kinds */
int b200profStop(void);              /* flushes everything in flight, then disables all kinds */
int b200profFlush(void);
uint64_t b200profKernels(b200prof_kernel_t* out, uint64_t max); /* returns how many exist */
uint64_t b200profMemops(b200prof_memop_t* out, uint64_t max);
uint64_t b200profApis(b200prof_api_t* out, uint64_t max);
uint64_t b200profDropped(void);      /* records CUPTI reported as dropped */
void b200profClear(void);
/* Writes <prefix>_kernel_trace.csv, <prefix>_memory_copy_trace.csv, <prefix>_cuda_api_trace.csv
 * (only the kinds that have records). Returns the number of files written, <0 on error. */
int b200profWriteCsv(const char* prefix);
const char* b200profLastError(void);

#ifdef __cplusplus
}
#endif

#endif /* B200COLL_PROF_H_ */
