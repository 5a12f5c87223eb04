// Instantiates the reducing kernels for one element type. Compiled once per type with
// -DB200_T=<type> -DB200_TN=<suffix> [-DB200_NVLS_OK=1] so the twelve types build in parallel.
#include <atomic>
#include "kernels.cuh"
#include "launch.h"

#define B200_CAT2(a, b) a##b
#define B200_CAT(a, b) B200_CAT2(a, b)

namespace b200 {

cudaError_t B200_CAT(launchLL_, B200_TN)(int op, int grid, cudaStream_t s, const DevComm& c, const LLArgs& a) {
  switch (op) {
    case ncclSum: kLLAllReduce<B200_T, OpSum><<<grid, kCollThreads, 0, s>>>(c, a); break;
    case ncclProd: kLLAllReduce<B200_T, OpProd><<<grid, kCollThreads, 0, s>>>(c, a); break;
    case ncclMax: kLLAllReduce<B200_T, OpMax><<<grid, kCollThreads, 0, s>>>(c, a); break;
    case ncclMin: kLLAllReduce<B200_T, OpMin><<<grid, kCollThreads, 0, s>>>(c, a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t B200_CAT(launchStaged_, B200_TN)(int op, bool nvls, int grid, cudaStream_t s, const DevComm& c, const CollArgs& a) {
  if (nvls) {
#ifdef B200_NVLS_OK
    if (op != ncclSum) return cudaErrorInvalidValue;
    kStagedReduce<B200_T, OpSum, true><<<grid, kCollThreads, 0, s>>>(c, a);  // switch-side adds need few registers: full-size CTAs
    return cudaGetLastError();
#else
    return cudaErrorInvalidValue;
#endif
  }
  // The peer-load kernels stage tiles in a shared-memory ring larger than the default limit.
  // The limit is a property of (function, device): a process that drives several GPUs (one thread per GPU) sets it on each.
  static std::atomic<bool> allowed[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !allowed[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(kStagedReduce<B200_T, OpSum, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kStagedReduce<B200_T, OpProd, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kStagedReduce<B200_T, OpMax, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kStagedReduce<B200_T, OpMin, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmemBytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) allowed[dev].store(true, std::memory_order_release);
  }
  switch (op) {
    case ncclSum: kStagedReduce<B200_T, OpSum, false><<<grid, kReduceThreads, kBulkSmemBytes, s>>>(c, a); break;
    case ncclProd: kStagedReduce<B200_T, OpProd, false><<<grid, kReduceThreads, kBulkSmemBytes, s>>>(c, a); break;
    case ncclMax: kStagedReduce<B200_T, OpMax, false><<<grid, kReduceThreads, kBulkSmemBytes, s>>>(c, a); break;
    case ncclMin: kStagedReduce<B200_T, OpMin, false><<<grid, kReduceThreads, kBulkSmemBytes, s>>>(c, a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace b200
