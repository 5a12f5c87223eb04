// Host-callable launchers of the collective kernels.
#pragma once

#include <cuda_runtime_api.h>

#include "device.h"

namespace b200 {

// `op` is one of ncclSum/ncclProd/ncclMax/ncclMin; Avg and PreMulSum arrive as Sum + scaleMode.
cudaError_t launchLLAllReduce(ncclDataType_t dt, int op, int grid, cudaStream_t s, const DevComm& c, const LLArgs& a);  // all-reduce and reduce-scatter (a.kind)
cudaError_t launchLLAllGather(int grid, cudaStream_t s, const DevComm& c, const LLArgs& a);
cudaError_t launchStagedReduce(ncclDataType_t dt, int op, bool nvls, int grid, cudaStream_t s, const DevComm& c, const CollArgs& a);
cudaError_t launchStagedCopy(bool nvls, int grid, cudaStream_t s, const DevComm& c, const CollArgs& a, int elemSize);
cudaError_t launchP2p(int grid, cudaStream_t s, const DevComm& c, const P2pArgs& a);
cudaError_t launchAllToAllDirect(int grid, cudaStream_t s, const DevComm& c, const A2aDirectArgs& a);
cudaError_t launchBarrier(cudaStream_t s, const DevComm& c);
cudaError_t launchWaitUnsetFlag(cudaStream_t s, const DevComm& c);
cudaError_t launchFill(void* dst, unsigned value, size_t bytes, cudaStream_t s);
cudaError_t launchCopy(void* dst, const void* src, size_t bytes, int grid, cudaStream_t s);
bool nvlsReducible(ncclDataType_t dt, int op);  // can the switch do this reduction?

#define B200_DECL_T(TN)                                                                                     \
  cudaError_t launchLL_##TN(int op, int grid, cudaStream_t s, const DevComm& c, const LLArgs& a);            \
  cudaError_t launchStaged_##TN(int op, bool nvls, int grid, cudaStream_t s, const DevComm& c, const CollArgs& a);
B200_DECL_T(i8) B200_DECL_T(u8) B200_DECL_T(i32) B200_DECL_T(u32) B200_DECL_T(i64) B200_DECL_T(u64)
B200_DECL_T(f16) B200_DECL_T(f32) B200_DECL_T(f64) B200_DECL_T(bf16) B200_DECL_T(e4m3) B200_DECL_T(e5m2)
#undef B200_DECL_T

}  // namespace b200
