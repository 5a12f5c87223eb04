// RMSNorm backward without any device allocation: the fp32 accumulator of the weight gradient is
// a file-scope device array instead of caller-provided memory. See no_alloc.h for who this is for
// and for the rules of use.
#include "no_alloc.h"

#include <cuda_bf16.h>
#include <stdio.h>

#include <mutex>

// The regular entry point (train_ops.cu); it accumulates the weight gradient into the fp32 buffer
// it is given, which here is the array below.
extern "C" int b200ops_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw, long long T, int H,
                                   cudaStream_t s);

namespace {

// The scratch. In host code this name is only a stand-in for the symbol, never a device address:
// the address kernels may use comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) float gDwScratch[B200OPS_NOALLOC_MAX_H];

constexpr int kMaxDevices = 64;
std::mutex gSetupMu;
float* gScratchAddr[kMaxDevices] = {};
thread_local char tlsError[256] = "";

// Device address of the array on the current device, looked up on the first call there.
float* scratchForCurrentDevice() {
  int dev = -1;
  cudaError_t ge = cudaGetDevice(&dev);
  if (ge != cudaSuccess) {
    snprintf(tlsError, sizeof(tlsError), "cudaGetDevice failed: %s", cudaGetErrorString(ge));
    (void)cudaGetLastError();
    return nullptr;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    snprintf(tlsError, sizeof(tlsError), "device %d is outside the %d devices this entry point keeps an address for", dev, kMaxDevices);
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(gSetupMu);
  if (!gScratchAddr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, gDwScratch);
    if (e != cudaSuccess || !p) {
      snprintf(tlsError, sizeof(tlsError), "cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      (void)cudaGetLastError();
      return nullptr;
    }
    gScratchAddr[dev] = static_cast<float*>(p);
  }
  return gScratchAddr[dev];
}

__global__ void clearScratch(float* scratch, int H) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) scratch[i] = 0.f;
}

__global__ void castScratch(const float* scratch, __nv_bfloat16* dw, int H) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) dw[i] = __float2bfloat16(scratch[i]);
}

}  // namespace

extern "C" int b200ops_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dwBf16, long long T, int H,
                                           cudaStream_t stream) {
  tlsError[0] = '\0';
  if (H <= 0 || H % 8 != 0 || H > B200OPS_NOALLOC_MAX_H) {
    snprintf(tlsError, sizeof(tlsError), "row width %d is not supported: it must be a multiple of 8 and at most %d (the size of the built-in scratch)", H,
             B200OPS_NOALLOC_MAX_H);
    return B200OPS_NOALLOC_ERR_TOO_LARGE;
  }
  float* scratch = scratchForCurrentDevice();
  if (!scratch) return B200OPS_NOALLOC_ERR_SETUP;
  const int blocks = (H + 255) / 256;
  clearScratch<<<blocks, 256, 0, stream>>>(scratch, H);  // the array still holds the previous call's gradient
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (T > 0) {
    int rc = b200ops_rmsnorm_bwd(dy, x, w, rstd, dx, scratch, T, H, stream);
    if (rc != 0) return rc;
  }
  castScratch<<<blocks, 256, 0, stream>>>(scratch, static_cast<__nv_bfloat16*>(dwBf16), H);
  return (int)cudaGetLastError();
}

extern "C" const char* b200ops_rmsnorm_bwd_noalloc_error(void) { return tlsError; }
