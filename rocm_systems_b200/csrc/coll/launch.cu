// Type dispatch and the type-agnostic kernels (copy collectives, send/recv, barrier, copy, fill).
#define B200_MISC_KERNELS 1
#include "kernels.cuh"
#include "launch.h"

namespace b200 {

bool nvlsReducible(ncclDataType_t dt, int op) {
  return op == ncclSum && (dt == ncclFloat32 || dt == ncclFloat16 || dt == ncclBfloat16);
}

#define B200_SWITCH_T(fn, ...)                                  \
  switch (dt) {                                                 \
    case ncclInt8: return fn##_i8(__VA_ARGS__);                 \
    case ncclUint8: return fn##_u8(__VA_ARGS__);                \
    case ncclInt32: return fn##_i32(__VA_ARGS__);               \
    case ncclUint32: return fn##_u32(__VA_ARGS__);              \
    case ncclInt64: return fn##_i64(__VA_ARGS__);               \
    case ncclUint64: return fn##_u64(__VA_ARGS__);              \
    case ncclFloat16: return fn##_f16(__VA_ARGS__);             \
    case ncclFloat32: return fn##_f32(__VA_ARGS__);             \
    case ncclFloat64: return fn##_f64(__VA_ARGS__);             \
    case ncclBfloat16: return fn##_bf16(__VA_ARGS__);           \
    case ncclFp8E4M3: return fn##_e4m3(__VA_ARGS__);            \
    case ncclFp8E5M2: return fn##_e5m2(__VA_ARGS__);            \
    default: return cudaErrorInvalidValue;                      \
  }

cudaError_t launchLLAllReduce(ncclDataType_t dt, int op, int grid, cudaStream_t s, const DevComm& c, const LLArgs& a) {
  B200_SWITCH_T(launchLL, op, grid, s, c, a)
}
cudaError_t launchStagedReduce(ncclDataType_t dt, int op, bool nvls, int grid, cudaStream_t s, const DevComm& c, const CollArgs& a) {
  B200_SWITCH_T(launchStaged, op, nvls, grid, s, c, a)
}

cudaError_t launchStagedCopy(bool nvls, int grid, cudaStream_t s, const DevComm& c, const CollArgs& a, int elemSize) {
  if (nvls) kStagedCopy<true><<<grid, kCollThreads, 0, s>>>(c, a, elemSize);
  else kStagedCopy<false><<<grid, kCollThreads, 0, s>>>(c, a, elemSize);
  return cudaGetLastError();
}

cudaError_t launchLLAllGather(int grid, cudaStream_t s, const DevComm& c, const LLArgs& a) {
  kLLAllGather<<<grid, kCollThreads, 0, s>>>(c, a);
  return cudaGetLastError();
}

cudaError_t launchP2p(int grid, cudaStream_t s, const DevComm& c, const P2pArgs& a) {
  kP2p<<<grid, kCollThreads, 0, s>>>(c, a);
  return cudaGetLastError();
}

// Waits on a flag word that nothing ever writes, so the wait budget runs out: the way the
// time-out path (status word, async error) is exercised without any rank misbehaving.
__global__ void kWaitUnsetFlag(const __grid_constant__ DevComm c) {
  const uint32_t* flag = (const uint32_t*)(c.ws[c.rank] + kWsUserFlagsOff + 48 * 1024 - 64);
  if (threadIdx.x == 0) waitGe(c, flag, 1u, WAIT_SHMEM, (uint32_t)c.rank);
}
cudaError_t launchWaitUnsetFlag(cudaStream_t s, const DevComm& c) {
  kWaitUnsetFlag<<<1, 32, 0, s>>>(c);
  return cudaGetLastError();
}

cudaError_t launchAllToAllDirect(int grid, cudaStream_t s, const DevComm& c, const A2aDirectArgs& a) {
  kAllToAllDirect<<<grid, kCollThreads, 0, s>>>(c, a);
  return cudaGetLastError();
}

cudaError_t launchBarrier(cudaStream_t s, const DevComm& c) {
  kBarrier<<<1, 32, 0, s>>>(c);
  return cudaGetLastError();
}

// Successors of the runtime's shader-blit copy and fill kernels
// (rocr-runtime/runtime/hsa-runtime/core/runtime/amd_blit_kernel.cpp:718-837): 16-byte vector
// body, narrower paths for unaligned ends.
__global__ void __launch_bounds__(kCollThreads) kCopy(char* dst, const char* src, size_t bytes) {
  size_t lo, hi;
  splitUnits((bytes + 15) >> 4, gridDim.x, blockIdx.x, lo, hi);
  if (lo >= hi) return;
  const size_t n = ((hi << 4) < bytes ? (hi << 4) : bytes) - (lo << 4);
  ctaCopy(dst + (lo << 4), src + (lo << 4), n);
}

__global__ void __launch_bounds__(kCollThreads) kFill(char* dst, unsigned value, size_t bytes) {
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, gn = (size_t)gridDim.x * blockDim.x;
  // Head bytes up to 16-byte alignment, vector body, tail bytes. `value` repeats every 4 bytes
  // counted from dst, so the byte written at offset o is byte (o & 3) of value.
  const size_t mis = (16 - ((uintptr_t)dst & 15)) & 15;
  const size_t head = mis < bytes ? mis : bytes;
  for (size_t o = gtid; o < head; o += gn) dst[o] = (char)(value >> (8 * (o & 3)));
  const size_t body = (bytes - head) >> 4;
  const unsigned sh = (unsigned)(head & 3) * 8;
  const unsigned rot = sh ? (value >> sh) | (value << (32 - sh)) : value;
  for (size_t i = gtid; i < body; i += gn) st16(dst + head + (i << 4), make_uint4(rot, rot, rot, rot));
  for (size_t o = head + (body << 4) + gtid; o < bytes; o += gn) dst[o] = (char)(value >> (8 * (o & 3)));
}

cudaError_t launchCopy(void* dst, const void* src, size_t bytes, int grid, cudaStream_t s) {
  if (bytes == 0) return cudaSuccess;
  if (grid <= 0) {
    size_t want = (bytes + (size_t)kCollThreads * 128 - 1) / ((size_t)kCollThreads * 128);
    grid = want > 296 ? 296 : (want < 1 ? 1 : (int)want);
  }
  kCopy<<<grid, kCollThreads, 0, s>>>((char*)dst, (const char*)src, bytes);
  return cudaGetLastError();
}

cudaError_t launchFill(void* dst, unsigned value, size_t bytes, cudaStream_t s) {
  if (bytes == 0) return cudaSuccess;
  size_t want = (bytes + (size_t)kCollThreads * 64 - 1) / ((size_t)kCollThreads * 64);
  int grid = want > 296 ? 296 : (want < 1 ? 1 : (int)want);
  kFill<<<grid, kCollThreads, 0, s>>>((char*)dst, value, bytes);
  return cudaGetLastError();
}

}  // namespace b200
