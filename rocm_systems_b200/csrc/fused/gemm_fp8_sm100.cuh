// Block-scaled fp8 (e4m3) GEMM main loop on the 5th-generation tensor cores, as a CTA-level routine with policy hooks:
//   C[M, N] = sum over 128-wide K blocks kb of  sA[kb][m] * sB[n / 128][kb] * (A8[m, kb] . B8[n, kb])
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
// the MMAs, warps 2..5 promote and, at the end of a tile, hand the fp32 tile to the policy.
// Tile order, operand readiness, where the activation scales come from and what happens to a finished
// tile are hooks of a policy object: the plain GEMM and the fused GEMM+collective kernels differ only there.
// Every wait is bounded.
#pragma once

#include <cuda_fp8.h>

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
  int* err;          // device word: 0, or the code of the first wait that gave up (gemm::ErrCode)
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

// Policy interface (all __device__):
//   void coord(int t, int tilesM, int tilesN, int& tm, int& tn)   tile order
//   bool valid(int tm, int tn)                                   false: the tile is skipped by every role
//   int bRow(int tm, int tn)                                     first row of the tile in the B tensor map
//   int scaleBOff(int tm, int tn)                                offset into p.sB of the tile's weight scales (one per K block)
//   bool waitTile(int tm, int tn, volatile int* err)             producer thread: the A rows of the tile are in place
//   bool epiBegin(int tm, volatile int* err)                     every epilogue thread, before the first scale of a tile is read
//   float scaleA(int kb, int row)                                activation scale of `row` for K block kb (row < M)
//   void emit(float (&acc)[BN], int tm, int tn, int q, int lane, uint8_t* sw)   epilogue warp q: the lane's row of the finished
//                                                                tile (row tm * BM + q * 32 + lane); sw: the warp's 8 KiB staging buffer
//   void tileDone(int tm, int tn, int q, int lane)               epilogue thread, after its rows of the tile are out
template <typename Policy>
__device__ __forceinline__ void gemmFp8Cta(const Params& p, Policy& pol, int cta, int nctas, uint8_t* smemRaw) {
  using namespace sm100;
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
        pol.coord(t, p.tilesM, p.tilesN, tm, tn);
        if (!pol.valid(tm, tn)) continue;
        if (!pol.waitTile(tm, tn, err)) { ok = false; break; }
        const int bRow = pol.bRow(tm, tn);
        for (int k = 0; k < kIters; k++) {
          if (!mbarWait(&empty[stage], phase ^ 1, err, gemm::ERR_PRODUCER_EMPTY)) { ok = false; break; }
          mbarArriveExpectTx(&full[stage], kStageBytes);
          tmaLoad2d(smemA + (size_t)stage * kABytes, &p.mapA, k * BK, tm * BM, &full[stage]);
          tmaLoad2d(smemB + (size_t)stage * kBBytes, &p.mapB, k * BK, bRow, &full[stage]);
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
        {
          int tm, tn;
          pol.coord(t, p.tilesM, p.tilesN, tm, tn);
          if (!pol.valid(tm, tn)) continue;
        }
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
      pol.coord(t, p.tilesM, p.tilesN, tm, tn);
      if (!pol.valid(tm, tn)) continue;
      if (!pol.epiBegin(tm, err)) { ok = false; break; }
      const int row = tm * BM + q * 32 + lane;
      float acc[BN];
#pragma unroll
      for (int i = 0; i < BN; i++) acc[i] = 0.f;
      for (int k = 0; k < kIters; k++) {
        const uint32_t b = blk & 1, bPhase = (blk >> 1) & 1;
        blk++;
        const float s = (row < p.M ? pol.scaleA(k, row) : 0.f) * __ldg(p.sB + (size_t)pol.scaleBOff(tm, tn) + k);
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
      pol.emit(acc, tm, tn, q, lane, epiStage + (size_t)q * kEpiBytesPerWarp);
      pol.tileDone(tm, tn, q, lane);
    }
  }
  tcFenceBefore();
  __syncthreads();
  if (warp == 1) tmemDealloc(tmem, kTmemCols);
}

// ---- the plain GEMM: banded order, nothing to wait for, C = bf16(acc) ------------------------------------
struct PlainPolicy8 {
  const Params& p;  // the kernel's __grid_constant__ parameter
  __device__ __forceinline__ void coord(int t, int tilesM, int tilesN, int& tm, int& tn) const { gemm::bandedCoord(t, tilesM, tilesN, tm, tn); }
  __device__ __forceinline__ bool valid(int, int) const { return true; }
  __device__ __forceinline__ int bRow(int, int tn) const { return tn * BN; }
  __device__ __forceinline__ int scaleBOff(int, int tn) const { return tn * p.kBlocks; }
  __device__ __forceinline__ bool waitTile(int, int, volatile int*) const { return true; }
  __device__ __forceinline__ bool epiBegin(int, volatile int*) const { return true; }
  __device__ __forceinline__ float scaleA(int kb, int row) const { return __ldg(p.sA + (size_t)kb * p.M + row); }
  __device__ __forceinline__ void emit(float (&acc)[BN], int tm, int tn, int q, int lane, uint8_t* sw) const {
    const int row0 = tm * BM + q * 32;
    storeTile(sw, lane, p.N - tn * BN, acc,
              [&](int r) -> __nv_bfloat16* { return row0 + r < p.M ? p.C + (size_t)(row0 + r) * p.ldc + (size_t)tn * BN : nullptr; });
  }
  __device__ __forceinline__ void tileDone(int, int, int, int) const {}
};

}  // namespace gemm8
}  // namespace b200
