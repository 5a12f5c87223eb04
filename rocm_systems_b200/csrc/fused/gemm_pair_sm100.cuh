// bf16 GEMM on CTA pairs (tcgen05 cta_group::2) with either operand K-major or MN-major:
//   C[M, N] = A * B^T,  A logical [M, K], B logical [N, K], fp32 accumulation, bf16 out.
// "K-major": the operand is stored [rows, K] row-major (the reduction index is contiguous). "MN-major": it is stored
// [K, rows] row-major (the row index is contiguous), which is how the operands of a backward pass lie in memory:
//   y  = x  w^T      A = x  (K-major)   B = w  (K-major)
//   dx = dy w        A = dy (K-major)   B = w  read as [N_red, K_out]: MN-major
//   dw = dy^T x      A = dy read as [T_red, N]: MN-major   B = x read as [T_red, K]: MN-major
// so no transposed copy of anything is ever made.
//
// Two CTAs of a cluster work on one 256 x BN output tile. Each loads its own 128 rows of A and its own half of the B
// tile (BN / 2 rows) with ordinary TMA tile loads into its own shared memory; the even CTA's elected thread issues one
// 256 x BN x 16 MMA per step that reads both halves and writes 128 accumulator rows into each CTA's tensor memory.
// Against one CTA per tile that halves the shared-memory traffic of B (three stages of 128 reduction steps fit). The byte count of
// both CTAs' loads lands on the even CTA's `full` barrier; the MMA thread's commits arrive on the `empty` barriers of both
// CTAs (one commit addressed to both) and, at the end of a tile, on both `accFull` barriers; the epilogue warps of both CTAs
// arrive on the even CTA's `accEmpty`. Four epilogue warps per CTA drain tensor memory through a swizzled staging buffer
// into 256-byte row segments while the next tile's main loop runs (two accumulators). Every wait is bounded; a CTA that
// gives up still reaches the cluster barriers at the end.
#pragma once

#include "gemm_sm100.cuh"

namespace b200 {
namespace gemm2 {

using gemm::BK;
using gemm::BM;
using gemm::kThreads;

// A stage holds 128 reduction steps (two TMA boxes of 64 per operand): eight MMAs per barrier round trip. With 64 the
// issuing thread spent as long on the wait / commit pair of a stage as the tensor cores on its four MMAs.
constexpr int kStages = 3;
constexpr int kSub = 2;                        // 64-wide reduction slices per stage
constexpr uint32_t kChunkBytes = 64 * BK * 2;  // one MN-major TMA box: 64 reduction rows of 64 elements

template <int BN> struct Cfg {
  static constexpr uint32_t kASub = BM * BK * 2;            // this CTA's 128 rows of A, 64 reduction steps
  static constexpr uint32_t kBSub = (BN / 2) * BK * 2;      // this CTA's half of the B tile, 64 reduction steps
  static constexpr uint32_t kABytes = kSub * kASub;
  static constexpr uint32_t kBBytes = kSub * kBSub;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kTmemCols = 2 * BN;
  static constexpr uint32_t kEpiBytesPerWarp = 32 * 128 * 2;
  static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 + 256 + 4 * kEpiBytesPerWarp;
};

struct Params {
  CUtensorMap mapA;  // K-major: [M, K], box {64, 128}.   MN-major: [K, M], box {64, 64}
  CUtensorMap mapB;  // K-major: [N, K], box {64, BN / 2}. MN-major: [K, N], box {64, 64}
  __nv_bfloat16* C;
  int ldc;
  int M, N, K;
  int tilesM, tilesN;  // tiles of 256 x BN
  int* err;
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1) gemmPairKernel(const __grid_constant__ Params p) {
  using C = Cfg<BN>;
  using namespace sm100;
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smemA = smem;
  uint8_t* smemB = smem + (size_t)kStages * C::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * C::kStageBytes);
  uint64_t* full = bars;                 // used in the even CTA only
  uint64_t* empty = bars + kStages;      // one set per CTA
  uint64_t* accFull = bars + 2 * kStages;   // one set per CTA
  uint64_t* accEmpty = accFull + 2;      // used in the even CTA only
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(accEmpty + 2);
  uint8_t* epiStage = reinterpret_cast<uint8_t*>(bars) + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cr = clusterCtaRank();  // 0: issues the MMAs; 1: its partner
  volatile int* err = p.err;

  if (threadIdx.x == 0) {
    prefetchTensorMap(&p.mapA);
    prefetchTensorMap(&p.mapB);
    for (int s = 0; s < kStages; s++) {
      mbarInit(&full[s], 1);
      mbarInit(&empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbarInit(&accFull[b], 1);
      mbarInit(&accEmpty[b], 8);  // four epilogue warps in each CTA of the pair
    }
    fenceBarrierInit();
  }
  if (warp == 1) {
    tmemAllocPair(tmemSlot, C::kTmemCols);
    tmemRelinquishPair();
  }
  tcFenceBefore();
  __syncthreads();
  clusterArrive();  // the partner's barriers exist before anything arrives on them
  clusterWait();
  tcFenceAfter();
  const uint32_t tmem = *tmemSlot;

  const int numTiles = p.tilesM * p.tilesN;
  const int kIters = (p.K + kSub * BK - 1) / (kSub * BK);
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < numTiles && ok; t += npairs) {
        int tm, tn;
        gemm::bandedCoord(t, p.tilesM, p.tilesN, tm, tn);
        const int aRow = tm * 2 * BM + (int)cr * BM;
        const int bRow = tn * BN + (int)cr * (BN / 2);
        for (int k = 0; k < kIters; k++) {
          if (!mbarWait(&empty[stage], phase ^ 1, err, gemm::ERR_PRODUCER_EMPTY)) { ok = false; break; }
          const uint32_t fullAddr = mapToCta(smemAddr(&full[stage]), 0);
          if (cr == 0) mbarArriveExpectTx(&full[stage], 2 * C::kStageBytes);  // both CTAs' bytes land here
          uint8_t* sa = smemA + (size_t)stage * C::kABytes;
          uint8_t* sb = smemB + (size_t)stage * C::kBBytes;
#pragma unroll
          for (int h = 0; h < kSub; h++) {
            const int k0 = (k * kSub + h) * BK;  // a slice that starts beyond K reads zeros
            if constexpr (A_MN) {
#pragma unroll
              for (int c = 0; c < BM / 64; c++) tmaLoad2dPair(sa + h * C::kASub + c * kChunkBytes, &p.mapA, aRow + c * 64, k0, fullAddr);
            } else {
              tmaLoad2dPair(sa + h * C::kASub, &p.mapA, k0, aRow, fullAddr);
            }
            if constexpr (B_MN) {
#pragma unroll
              for (int c = 0; c < BN / 2 / 64; c++) tmaLoad2dPair(sb + h * C::kBSub + c * kChunkBytes, &p.mapB, bRow + c * 64, k0, fullAddr);
            } else {
              tmaLoad2dPair(sb + h * C::kBSub, &p.mapB, k0, bRow, fullAddr);
            }
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok && cr == 0)
        for (int s = 0; s < kStages; s++) mbarWait(&full[s], 0, err, 0, 2000u);  // let loads in flight land
    }
  } else if (warp == 1) {
    if (lane == 0 && cr == 0) {
      constexpr uint32_t idesc = instrDescMajor(2 * BM, BN, 1 /*bf16*/, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = pair; t < numTiles && ok; t += npairs) {
        const int b = it & 1;
        const uint32_t accPhase = (it >> 1) & 1;
        it++;
        if (!mbarWait(&accEmpty[b], accPhase ^ 1, err, gemm::ERR_MMA_ACC_EMPTY)) { ok = false; break; }
        tcFenceAfter();
        const uint32_t d = tmem + (uint32_t)b * BN;
        for (int k = 0; k < kIters; k++) {
          if (!mbarWait(&full[stage], phase, err, gemm::ERR_MMA_FULL)) { ok = false; break; }
          tcFenceAfter();
          const uint32_t aAddr = smemAddr(smemA + (size_t)stage * C::kABytes);
          const uint32_t bAddr = smemAddr(smemB + (size_t)stage * C::kBBytes);
#pragma unroll
          for (int h = 0; h < kSub; h++) {
#pragma unroll
            for (int kk = 0; kk < BK / 16; kk++) {
              // 16 reduction steps: 32 bytes along a K-major row, 16 rows of 128 bytes in an MN-major tile
              const uint32_t ah = aAddr + h * C::kASub, bh = bAddr + h * C::kBSub;
              const uint64_t da = A_MN ? smemDescSw128Mn(ah + kk * 2048, kChunkBytes) : smemDescSw128(ah + kk * 32);
              const uint64_t db = B_MN ? smemDescSw128Mn(bh + kk * 2048, kChunkBytes) : smemDescSw128(bh + kk * 32);
              mmaF16Pair(d, da, db, idesc, (k | h | kk) != 0);
            }
          }
          mmaCommitBoth(smemAddr(&empty[stage]));  // the stage is free in both CTAs once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) mmaCommitBoth(smemAddr(&accFull[b]));
      }
    }
  } else {
    const int q = warp & 3;
    int it = 0;
    bool ok = true;
    for (int t = pair; t < numTiles && ok; t += npairs) {
      int tm, tn;
      gemm::bandedCoord(t, p.tilesM, p.tilesN, tm, tn);
      const int b = it & 1;
      const uint32_t accPhase = (it >> 1) & 1;
      it++;
      if (!mbarWait(&accFull[b], accPhase, err, gemm::ERR_EPI_ACC_FULL)) { ok = false; break; }
      tcFenceAfter();
      const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * BN);
      const int row0 = tm * 2 * BM + (int)cr * BM + q * 32;
      gemm::drainStaged(
          epiStage + (size_t)q * C::kEpiBytesPerWarp, lane, BN, p.N - tn * BN,
          [&](int c, uint32_t(&acc)[32]) {
            tmemLoad32(taddr + c * 32, acc);
            tmemLoadWait();
          },
          [&](int r) -> __nv_bfloat16* { return row0 + r < p.M ? p.C + (size_t)(row0 + r) * p.ldc + (size_t)tn * BN : nullptr; });
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArriveCluster(mapToCta(smemAddr(&accEmpty[b]), 0));
    }
  }
  tcFenceBefore();
  __syncthreads();
  clusterArrive();  // no arrival may land on a CTA that has left, and no MMA may read the shared memory of one
  clusterWait();
  if (warp == 1) tmemDeallocPair(tmem, C::kTmemCols);
}

}  // namespace gemm2
}  // namespace b200
