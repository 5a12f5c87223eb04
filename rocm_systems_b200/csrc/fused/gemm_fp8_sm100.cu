// Block-scaled fp8 (e4m3) GEMM (main loop in gemm_fp8_sm100.cuh) as a plain kernel, and the quantisers that feed it.
#include "gemm_fp8_sm100.cuh"
#include "gemm_host.h"

namespace b200 {
namespace gemm8 {

__global__ void __launch_bounds__(kThreads, 1) gemmFp8BlockKernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t smemRaw[];
  PlainPolicy8 pol{p};
  gemmFp8Cta(p, pol, blockIdx.x, gridDim.x, smemRaw);
}

// ---- quantisers ------------------------------------------------------------------------------------------------
// Activations: one scale per row and 128 channels. A warp takes a row; lane l holds channels (32 j + l) * 8 .. + 8 of
// round j, so a half-warp is one 128-channel group.
__global__ void __launch_bounds__(256) quantRows1x128(const __nv_bfloat16* x, uint8_t* q, float* s, int M, int K, int ldx, int ldq, int lds) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) return;
  const int groups = K / 128;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * ldx);
  uint2* qr = reinterpret_cast<uint2*>(q + (size_t)row * ldq);
  for (int j = 0; j * 2 < groups; j++) {
    const int g = j * 2 + (lane >> 4);
    const bool live = g < groups;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (live) raw = xr[j * 32 + lane];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float f[8];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float2 pr = __bfloat1622float2(h[i]);
      f[2 * i] = pr.x;
      f[2 * i + 1] = pr.y;
      amax = fmaxf(amax, fmaxf(fabsf(pr.x), fabsf(pr.y)));
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fmaxf(amax, 1e-10f) * (1.f / 448.f);
    uint32_t w[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const __nv_fp8x4_e4m3 p4(make_float4(__fdiv_rn(f[4 * i], scale), __fdiv_rn(f[4 * i + 1], scale), __fdiv_rn(f[4 * i + 2], scale), __fdiv_rn(f[4 * i + 3], scale)));
      w[i] = *reinterpret_cast<const uint32_t*>(&p4);
    }
    if (live) {
      qr[j * 32 + lane] = make_uint2(w[0], w[1]);
      if ((lane & 15) == 0) s[(size_t)g * lds + row] = scale;
    }
  }
}

// Weights: one scale per 128 x 128 block. One CTA of 256 threads per block; thread t holds 8 channels of rows
// (t / 16) + 16 i, i = 0..7.
__global__ void __launch_bounds__(256) quantBlocks128x128(const __nv_bfloat16* w, uint8_t* q, float* s, int N, int K, int ldw, int ldq) {
  __shared__ float red[8];
  const int kb = blockIdx.x, nb = blockIdx.y;
  const int t = threadIdx.x, sub = t & 15, r0 = t >> 4;
  uint4 raw[8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int row = nb * 128 + r0 + 16 * i;
    raw[i] = make_uint4(0, 0, 0, 0);
    if (row < N) raw[i] = *reinterpret_cast<const uint4*>(w + (size_t)row * ldw + (size_t)kb * 128 + sub * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float2 pr = __bfloat1622float2(h[e]);
      amax = fmaxf(amax, fmaxf(fabsf(pr.x), fabsf(pr.y)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((t & 31) == 0) red[t >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
  const float scale = fmaxf(amax, 1e-10f) * (1.f / 448.f);
  if (t == 0) s[(size_t)nb * gridDim.x + kb] = scale;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int row = nb * 128 + r0 + 16 * i;
    if (row >= N) continue;
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
    float f[8];
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float2 pr = __bfloat1622float2(h[e]);
      f[2 * e] = pr.x;
      f[2 * e + 1] = pr.y;
    }
    uint32_t o[2];
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const __nv_fp8x4_e4m3 p4(make_float4(__fdiv_rn(f[4 * e], scale), __fdiv_rn(f[4 * e + 1], scale), __fdiv_rn(f[4 * e + 2], scale), __fdiv_rn(f[4 * e + 3], scale)));
      o[e] = *reinterpret_cast<const uint32_t*>(&p4);
    }
    *reinterpret_cast<uint2*>(q + (size_t)row * ldq + (size_t)kb * 128 + sub * 8) = make_uint2(o[0], o[1]);
  }
}

}  // namespace gemm8
}  // namespace b200

using namespace b200;

extern "C" {

// q[M, K] (e4m3, row stride ldq bytes) and s[K / 128][lds] from x[M, K] (bf16, row stride ldx elements). K % 128 == 0.
// lds >= M is the row stride of the scale table: a rank that owns rows [r0, r0 + M) of a larger matrix passes the table's
// full width and s + r0.
int b200ops_quant_e4m3_1x128_strided(const void* x, void* q, float* s, int M, int K, int ldx, int ldq, int lds, cudaStream_t st) {
  if (M <= 0 || K <= 0) return 0;
  if ((K & 127) || (ldx & 7) || (ldq & 7) || lds < M || ((uintptr_t)x & 15) || ((uintptr_t)q & 7)) return (int)cudaErrorInvalidValue;
  gemm8::quantRows1x128<<<(M + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, s, M, K, ldx, ldq, lds);
  return (int)cudaGetLastError();
}
int b200ops_quant_e4m3_1x128(const void* x, void* q, float* s, int M, int K, int ldx, int ldq, cudaStream_t st) {
  return b200ops_quant_e4m3_1x128_strided(x, q, s, M, K, ldx, ldq, M, st);
}

// q[N, K] (e4m3) and s[ceil(N / 128)][K / 128] from w[N, K] (bf16). K % 128 == 0.
int b200ops_quant_e4m3_128x128(const void* w, void* q, float* s, int N, int K, int ldw, int ldq, cudaStream_t st) {
  if (N <= 0 || K <= 0) return 0;
  if ((K & 127) || (ldw & 7) || (ldq & 7) || ((uintptr_t)w & 15) || ((uintptr_t)q & 7)) return (int)cudaErrorInvalidValue;
  dim3 grid(K / 128, (N + 127) / 128);
  gemm8::quantBlocks128x128<<<grid, 256, 0, st>>>((const __nv_bfloat16*)w, (uint8_t*)q, s, N, K, ldw, ldq);
  return (int)cudaGetLastError();
}

// C[M, N] (bf16, ldc) = block-scaled A8[M, K] (lda bytes) * B8[N, K]^T (ldb bytes); sA [K / 128][M], sB [ceil(N / 128)][K / 128].
int b200ops_gemm_fp8_block_tn(const void* A8, const float* sA, const void* B8, const float* sB, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                              int maxCtas, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 127) || ((uintptr_t)C & 15) || (ldc & 7)) return (int)cudaErrorInvalidValue;
  gemm8::Params p{};
  if (!gemm::makeTileMap(&p.mapA, A8, M, K, lda, gemm::BM, 1) || !gemm::makeTileMap(&p.mapB, B8, N, K, ldb, gemm8::BN, 1)) return (int)cudaErrorInvalidValue;
  p.sA = sA;
  p.sB = sB;
  p.C = (__nv_bfloat16*)C;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.tilesM = (M + gemm::BM - 1) / gemm::BM;
  p.tilesN = (N + gemm8::BN - 1) / gemm8::BN;
  p.kBlocks = K / 128;
  p.err = gemm::errWord();
  if (!p.err) return (int)cudaErrorMemoryAllocation;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm8::gemmFp8BlockKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm8::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured[dev] = true;
  }
  int ctas = gemm::smCount();
  if (maxCtas > 0 && maxCtas < ctas) ctas = maxCtas;
  const int tiles = p.tilesM * p.tilesN;
  if (tiles < ctas) ctas = tiles;
  gemm8::gemmFp8BlockKernel<<<ctas, gemm8::kThreads, gemm8::kSmemBytes, st>>>(p);
  return (int)cudaGetLastError();
}

}  // extern "C"
