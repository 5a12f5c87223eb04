// Block-scaled fp8 (e4m3) GEMM on the 5th-generation tensor cores, and the quantisers that feed it:
//   C[M, N] (bf16) = sum over 128-wide K blocks kb of  sA[kb][m] * sB[n / 128][kb] * (A8[m, kb] . B8[n, kb])
// A8 [M, K] and B8 [N, K] are e4m3, both K-major; activations carry one fp32 scale per row and 128
// channels (stored block-major, [K / 128][M], so a warp reads the scales of its 32 rows in one go),
// weights one scale per 128 x 128 block ([ceil(N / 128)][K / 128]).
//
// Structure of the bf16 kernel (gemm_sm100.cuh) with one difference: the tensor cores cannot apply a
// scale that changes along K, so each 128-wide K block is multiplied into a fresh accumulator in
// tensor memory (kind::f8f6f4, four K=32 instructions) and the four epilogue warps fold it into
// fp32 registers with the block's scale while the next block is being multiplied into the other
// accumulator. Per K block a CTA moves 32 KiB through shared memory and 64 KiB out of tensor memory,
// both below what the 4.2 MFLOP of tensor work take, so the promotion is hidden.
// Warp 0 feeds shared memory by TMA (6 stages of 128 x 128 A + 128 x 128 B bytes), warp 1 issues
// the MMAs, warps 2..5 promote and, at the end of a tile, write bf16 rows through a swizzled staging
// buffer. Every wait is bounded.
#include <cuda_fp8.h>

#include "gemm_host.h"
#include "gemm_sm100.cuh"

namespace b200 {
namespace gemm8 {

using gemm::BM;
using gemm::kThreads;
constexpr int BN = 128;
constexpr int BK = 128;  // elements and bytes: one 128-byte swizzle row
constexpr int kStages = 6;
constexpr uint32_t kABytes = BM * BK;
constexpr uint32_t kBBytes = BN * BK;
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kTmemCols = 2 * BN;
constexpr uint32_t kEpiBytesPerWarp = 32 * 128 * 2;
constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 + 256 + 4 * kEpiBytesPerWarp;

struct Params {
  CUtensorMap mapA;  // [M, K] bytes, box {128, BM}, 128-byte swizzle
  CUtensorMap mapB;  // [N, K] bytes, box {128, BN}
  const float* sA;   // [kBlocks][M]
  const float* sB;   // [tilesN][kBlocks]
  __nv_bfloat16* C;
  int M, N, K, ldc;
  int tilesM, tilesN, kBlocks;
  int* err;
};

// One epilogue warp's 32 rows x 128 columns, fp32 registers -> bf16 -> swizzled staging -> 256-byte row segments.
template <typename RowPtr>
__device__ __forceinline__ void storeTile(uint8_t* sw, int lane, int colLimit, const float (&acc)[BN], RowPtr rowPtr) {
#pragma unroll
  for (int j = 0; j < 16; j++) {  // 16-byte chunk j of the lane's 256-byte row: columns 8j .. 8j+7
    uint4 o;
    uint32_t* ow = &o.x;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __nv_bfloat162 h = __floats2bfloat162_rn(acc[j * 8 + 2 * i], acc[j * 8 + 2 * i + 1]);
      ow[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(sw + lane * 256 + ((j ^ (lane & 7)) << 4)) = o;
  }
  __syncwarp();
  const int sub = lane & 15, half = lane >> 4;
  const int validChunks = max(0, min(16, colLimit / 8));
#pragma unroll 1
  for (int r2 = 0; r2 < 32; r2 += 2) {
    const int r = r2 + half;
    __nv_bfloat16* dst = rowPtr(r);
    if (dst != nullptr && sub < validChunks) *reinterpret_cast<uint4*>(dst + sub * 8) = *reinterpret_cast<const uint4*>(sw + r * 256 + ((sub ^ (r & 7)) << 4));
  }
  const int tailStart = validChunks * 8, tailEnd = min(colLimit, BN);
  if (tailStart < tailEnd) {  // fewer than 8 columns left at the right edge of C
    __nv_bfloat16* dst = rowPtr(lane);
    if (dst != nullptr)
      for (int col = tailStart; col < tailEnd; col++) dst[col] = reinterpret_cast<const __nv_bfloat16*>(sw + lane * 256 + (((col >> 3) ^ (lane & 7)) << 4))[col & 7];
  }
  __syncwarp();
}

__global__ void __launch_bounds__(kThreads, 1) gemmFp8BlockKernel(const __grid_constant__ Params p) {
  using namespace sm100;
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smemA = smem;
  uint8_t* smemB = smem + (size_t)kStages * kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* partFull = bars + 2 * kStages;
  uint64_t* partEmpty = partFull + 2;
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(partEmpty + 2);
  uint8_t* epiStage = reinterpret_cast<uint8_t*>(bars) + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, nctas = gridDim.x;
  volatile int* err = p.err;

  if (threadIdx.x == 0) {
    prefetchTensorMap(&p.mapA);
    prefetchTensorMap(&p.mapB);
    for (int s = 0; s < kStages; s++) {
      mbarInit(&full[s], 1);
      mbarInit(&empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbarInit(&partFull[b], 1);
      mbarInit(&partEmpty[b], 4);  // one arrival per epilogue warp
    }
    fenceBarrierInit();
  }
  if (warp == 1) {
    tmemAlloc(tmemSlot, kTmemCols);
    tmemRelinquish();
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmem = *tmemSlot;
  const int numTiles = p.tilesM * p.tilesN;
  const int kIters = p.kBlocks;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cta; t < numTiles && ok; t += nctas) {
        int tm, tn;
        gemm::bandedCoord(t, p.tilesM, p.tilesN, tm, tn);
        for (int k = 0; k < kIters; k++) {
          if (!mbarWait(&empty[stage], phase ^ 1, err, gemm::ERR_PRODUCER_EMPTY)) { ok = false; break; }
          mbarArriveExpectTx(&full[stage], kStageBytes);
          tmaLoad2d(smemA + (size_t)stage * kABytes, &p.mapA, k * BK, tm * BM, &full[stage]);
          tmaLoad2d(smemB + (size_t)stage * kBBytes, &p.mapB, k * BK, tn * BN, &full[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok)
        for (int s = 0; s < kStages; s++) mbarWait(&full[s], 0, err, 0, 2000u);  // let loads in flight land
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instrDesc(BM, BN, 0 /*e4m3*/);
      int stage = 0;
      uint32_t phase = 0, blk = 0;
      bool ok = true;
      for (int t = cta; t < numTiles && ok; t += nctas) {
        for (int k = 0; k < kIters; k++) {
          const uint32_t b = blk & 1, bPhase = (blk >> 1) & 1;
          blk++;
          if (!mbarWait(&partEmpty[b], bPhase ^ 1, err, gemm::ERR_MMA_ACC_EMPTY)) { ok = false; break; }
          if (!mbarWait(&full[stage], phase, err, gemm::ERR_MMA_FULL)) { ok = false; break; }
          tcFenceAfter();
          const uint32_t d = tmem + b * BN;
          const uint32_t aAddr = smemAddr(smemA + (size_t)stage * kABytes);
          const uint32_t bAddr = smemAddr(smemB + (size_t)stage * kBBytes);
#pragma unroll
          for (int kk = 0; kk < BK / 32; kk++) mmaF8(d, smemDescSw128(aAddr + kk * 32), smemDescSw128(bAddr + kk * 32), idesc, kk != 0);
          mmaCommit(&empty[stage]);   // the stage is free once these MMAs have read it
          mmaCommit(&partFull[b]);    // and the block's product is complete
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    const int q = warp & 3;  // the quarter of tensor-memory lanes this warp may read
    uint32_t blk = 0;
    bool ok = true;
    for (int t = cta; t < numTiles && ok; t += nctas) {
      int tm, tn;
      gemm::bandedCoord(t, p.tilesM, p.tilesN, tm, tn);
      const int row = tm * BM + q * 32 + lane;
      float acc[BN];
#pragma unroll
      for (int i = 0; i < BN; i++) acc[i] = 0.f;
      for (int k = 0; k < kIters; k++) {
        const uint32_t b = blk & 1, bPhase = (blk >> 1) & 1;
        blk++;
        const float s = (row < p.M ? __ldg(p.sA + (size_t)k * p.M + row) : 0.f) * __ldg(p.sB + (size_t)tn * p.kBlocks + k);
        if (!mbarWait(&partFull[b], bPhase, err, gemm::ERR_EPI_ACC_FULL)) { ok = false; break; }
        tcFenceAfter();
        const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + b * BN;
#pragma unroll
        for (int c = 0; c < BN / 32; c++) {
          uint32_t x[32];
          tmemLoad32(taddr + c * 32, x);
          tmemLoadWait();
#pragma unroll
          for (int i = 0; i < 32; i++) acc[c * 32 + i] = fmaf(s, __uint_as_float(x[i]), acc[c * 32 + i]);
        }
        tcFenceBefore();
        __syncwarp();
        if (lane == 0) mbarArrive(&partEmpty[b]);
      }
      if (!ok) break;
      const int row0 = tm * BM + q * 32;
      storeTile(epiStage + (size_t)q * kEpiBytesPerWarp, lane, p.N - tn * BN, acc,
                [&](int r) -> __nv_bfloat16* { return row0 + r < p.M ? p.C + (size_t)(row0 + r) * p.ldc + (size_t)tn * BN : nullptr; });
    }
  }
  tcFenceBefore();
  __syncthreads();
  if (warp == 1) tmemDealloc(tmem, kTmemCols);
}

// ---- quantisers ------------------------------------------------------------------------------------------------
// Activations: one scale per row and 128 channels. A warp takes a row; lane l holds channels (32 j + l) * 8 .. + 8 of
// round j, so a half-warp is one 128-channel group.
__global__ void __launch_bounds__(256) quantRows1x128(const __nv_bfloat16* x, uint8_t* q, float* s, int M, int K, int ldx, int ldq) {
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
    const float scale = fmaxf(amax, 1e-10f) / 448.f;
    const float inv = 1.f / scale;
    uint32_t w[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const __nv_fp8x4_e4m3 p4(make_float4(f[4 * i] * inv, f[4 * i + 1] * inv, f[4 * i + 2] * inv, f[4 * i + 3] * inv));
      w[i] = *reinterpret_cast<const uint32_t*>(&p4);
    }
    if (live) {
      qr[j * 32 + lane] = make_uint2(w[0], w[1]);
      if ((lane & 15) == 0) s[(size_t)g * M + row] = scale;
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
  const float scale = fmaxf(amax, 1e-10f) / 448.f;
  const float inv = 1.f / scale;
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
      const __nv_fp8x4_e4m3 p4(make_float4(f[4 * e] * inv, f[4 * e + 1] * inv, f[4 * e + 2] * inv, f[4 * e + 3] * inv));
      o[e] = *reinterpret_cast<const uint32_t*>(&p4);
    }
    *reinterpret_cast<uint2*>(q + (size_t)row * ldq + (size_t)kb * 128 + sub * 8) = make_uint2(o[0], o[1]);
  }
}

}  // namespace gemm8
}  // namespace b200

using namespace b200;

extern "C" {

// q[M, K] (e4m3, row stride ldq bytes) and s[K / 128][M] from x[M, K] (bf16, row stride ldx elements). K % 128 == 0.
int b200ops_quant_e4m3_1x128(const void* x, void* q, float* s, int M, int K, int ldx, int ldq, cudaStream_t st) {
  if (M <= 0 || K <= 0) return 0;
  if ((K & 127) || (ldx & 7) || (ldq & 7) || ((uintptr_t)x & 15) || ((uintptr_t)q & 7)) return (int)cudaErrorInvalidValue;
  gemm8::quantRows1x128<<<(M + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, s, M, K, ldx, ldq);
  return (int)cudaGetLastError();
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
  gemm8::gemmFp8BlockKernel<<<ctas, gemm::kThreads, gemm8::kSmemBytes, st>>>(p);
  return (int)cudaGetLastError();
}

}  // extern "C"
