// Block-scaled fp8 (e4m3) GEMM main loop on the 5th-generation tensor cores, as a CTA-level routine with policy hooks:
//   C[M, N] = sum over 128-wide K blocks kb of  sA[kb][m] * sB[n / 128][kb] * (A8[m, kb] . B8[n, kb])
// A8 [M, K] and B8 [N, K] are e4m3, both K-major; activations carry one fp32 scale per row and 128
// channels (stored block-major, [K / 128][M], so a warp reads the scales of its 32 rows in one go),
// weights one scale per 128 x 128 block ([ceil(N / 128)][K / 128]).
//
// Structure of the bf16 kernel (gemm_sm100.cuh) with one difference: the tensor cores cannot apply a
// scale that changes along K, so each 128-wide K block is multiplied into a fresh accumulator in
// tensor memory (kind::f8f6f4, four K=32 instructions) and EIGHT epilogue warps fold it into
// fp32 registers with the block's scale while the next blocks are being multiplied into the other
// accumulators (four partial products of 128 columns fill the 512 columns of tensor memory, which hides the latency of the
// commit -> epilogue -> release round trip). Two warps share each quarter of the tensor-memory lanes and split its 128 columns
// (warp pair member h takes columns [32h, 32h+32) and [64+32h, 64+32h+32), so that with SwiGLU weights
// interleaved 64 gate / 64 up per tile every thread holds matching gate and up values): per block a
// thread issues two 32-column loads, waits once and does 64 FMAs. With four warps and 128 columns per
// thread (four loads, each followed by a wait) the promotion took twice as long as the block's MMAs and
// the tensor pipe was 18 % busy.
// Warp 0 feeds shared memory by TMA (3 stages of two K blocks: 2 x (128 x 128 A + 128 x 128 B) bytes), warp 1 issues
// the MMAs, warps 2..9 promote and, at the end of a tile, hand their part of the fp32 tile to the policy.
// Tile order, operand readiness, where the activation scales come from and what happens to a finished
// tile are hooks of a policy object: the plain GEMM and the fused GEMM+collective kernels differ only there.
// Every wait is bounded.
#pragma once

#include <cuda_fp8.h>

#include "gemm_sm100.cuh"

namespace b200 {
namespace gemm8 {

using gemm::BM;
constexpr int kThreads = 320;       // TMA warp, MMA warp, eight epilogue warps
constexpr int kEpiThreads = 256;
constexpr int BN = 128;
constexpr int kAccCols = 64;        // accumulator columns per epilogue thread
constexpr int BK = 128;  // elements and bytes: one 128-byte swizzle row
// A stage, a barrier round trip and a commit cover a GROUP of two K blocks: the issuing thread pays a few hundred cycles
// per tcgen05.commit, which with one block per commit (and a second commit for the accumulator) was several times the
// 256 cycles the block's four MMAs take. One commit per group now tells both the producer (the stage is free) and the
// epilogue warps (the group's two partial products are complete).
constexpr int kGroup = 2;
constexpr int kStages = 3;
constexpr uint32_t kABlock = BM * BK;
constexpr uint32_t kBBlock = BN * BK;
constexpr uint32_t kABytes = kGroup * kABlock;
constexpr uint32_t kBBytes = kGroup * kBBlock;
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr int kAccBufs = 4;             // partial products in flight in tensor memory (two groups of two): all 512 columns
constexpr int kAccGroups = kAccBufs / kGroup;
constexpr uint32_t kTmemCols = kAccBufs * BN;
constexpr uint32_t kEpiBytesPerWarp = 32 * kAccCols * 2;  // 32 rows x 64 bf16 columns staged per epilogue warp
constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 + 256 + 8 * kEpiBytesPerWarp;

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

// Output column of accumulator element i of an epilogue thread whose warp is member h of its pair.
__device__ __forceinline__ int accCol(int i, int h) { return (i < 32 ? 0 : 64) + h * 32 + (i & 31); }

// One epilogue warp's 32 rows x NC columns (NC = 64: the thread's two 32-column groups, which lie 64 columns apart in
// the tile; NC = 32: one group, as after SwiGLU), fp32 registers -> bf16 -> swizzled staging -> 16-byte pieces of rows,
// 64 contiguous bytes per group. rowPtr(r) is the address of output column 0 OF THE TILE in the warp's r-th row (nullptr
// skips the row); group g of the staged row goes to columns gCol(g) .. gCol(g) + 32; colLimit: columns of the tile that exist.
template <int NC, typename RowPtr, typename GroupCol>
__device__ __forceinline__ void storeCols(uint8_t* sw, int lane, int colLimit, const float* acc, RowPtr rowPtr, GroupCol gCol) {
  constexpr int kChunks = NC / 8;  // 16-byte chunks per staged row
#pragma unroll
  for (int j = 0; j < kChunks; j++) {
    uint4 o;
    uint32_t* ow = &o.x;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __nv_bfloat162 h = __floats2bfloat162_rn(acc[j * 8 + 2 * i], acc[j * 8 + 2 * i + 1]);
      ow[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(sw + lane * (NC * 2) + ((j ^ (lane & (kChunks - 1))) << 4)) = o;
  }
  __syncwarp();
  constexpr int kRowsPerPass = 32 / kChunks;
  const int sub = lane % kChunks, rsel = lane / kChunks;
#pragma unroll 1
  for (int r0 = 0; r0 < 32; r0 += kRowsPerPass) {
    const int r = r0 + rsel;
    __nv_bfloat16* dst = rowPtr(r);
    const int col = gCol(sub >> 2) + (sub & 3) * 8;
    if (dst == nullptr || col >= colLimit) continue;
    const uint4 v = *reinterpret_cast<const uint4*>(sw + r * (NC * 2) + ((sub ^ (r & (kChunks - 1))) << 4));
    if (col + 8 <= colLimit) {
      *reinterpret_cast<uint4*>(dst + col) = v;
    } else {  // fewer than 8 columns left at the right edge of the output
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
      for (int k = 0; col + k < colLimit; k++) dst[col + k] = e[k];
    }
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
//   void emit(float (&acc)[kAccCols], int tm, int tn, int q, int h, int lane, uint8_t* sw)
//                                                                epilogue warp (q, h): the lane's row of the finished tile (row tm * BM +
//                                                                q * 32 + lane), columns accCol(i, h); sw: the warp's 4 KiB staging buffer
//   void tileDone(int tm, int tn, int q, int h, int lane)        epilogue thread, after its part of the tile is out
template <typename Policy>
__device__ __forceinline__ void gemmFp8Cta(const Params& p, Policy& pol, int cta, int nctas, uint8_t* smemRaw) {
  using namespace sm100;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smemA = smem;
  uint8_t* smemB = smem + (size_t)kStages * kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * kStageBytes);
  uint64_t* full = bars;                    // loads of a stage have landed
  uint64_t* done = bars + kStages;          // the MMAs of the group in a stage are complete: stage free AND products ready
  uint64_t* partEmpty = bars + 2 * kStages; // the epilogue warps have folded a group of accumulators
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(partEmpty + kAccGroups);
  uint8_t* epiStage = reinterpret_cast<uint8_t*>(bars) + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* err = p.err;

  if (threadIdx.x == 0) {
    prefetchTensorMap(&p.mapA);
    prefetchTensorMap(&p.mapB);
    for (int s = 0; s < kStages; s++) {
      mbarInit(&full[s], 1);
      mbarInit(&done[s], 1);
    }
    for (int b = 0; b < kAccGroups; b++) mbarInit(&partEmpty[b], 8);  // one arrival per epilogue warp
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
  const int kGroups = (p.kBlocks + kGroup - 1) / kGroup;  // a last, half-filled group multiplies zeros (loads beyond K read zeros)

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
        for (int g = 0; g < kGroups; g++) {
          if (!mbarWait(&done[stage], phase ^ 1, err, gemm::ERR_PRODUCER_EMPTY)) { ok = false; break; }
          mbarArriveExpectTx(&full[stage], kStageBytes);
#pragma unroll
          for (int j = 0; j < kGroup; j++) {
            tmaLoad2d(smemA + (size_t)stage * kABytes + j * kABlock, &p.mapA, (g * kGroup + j) * BK, tm * BM, &full[stage]);
            tmaLoad2d(smemB + (size_t)stage * kBBytes + j * kBBlock, &p.mapB, (g * kGroup + j) * BK, bRow, &full[stage]);
          }
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
      uint32_t phase = 0, grp = 0;
      bool ok = true;
      for (int t = cta; t < numTiles && ok; t += nctas) {
        {
          int tm, tn;
          pol.coord(t, p.tilesM, p.tilesN, tm, tn);
          if (!pol.valid(tm, tn)) continue;
        }
        for (int g = 0; g < kGroups; g++) {
          const uint32_t ab = grp % kAccGroups, abPhase = (grp / kAccGroups) & 1;
          grp++;
          if (!mbarWait(&partEmpty[ab], abPhase ^ 1, err, gemm::ERR_MMA_ACC_EMPTY)) { ok = false; break; }
          if (!mbarWait(&full[stage], phase, err, gemm::ERR_MMA_FULL)) { ok = false; break; }
          tcFenceAfter();
#pragma unroll
          for (int j = 0; j < kGroup; j++) {
            const uint32_t d = tmem + (ab * kGroup + j) * BN;
            const uint32_t aAddr = smemAddr(smemA + (size_t)stage * kABytes + j * kABlock);
            const uint32_t bAddr = smemAddr(smemB + (size_t)stage * kBBytes + j * kBBlock);
#pragma unroll
            for (int kk = 0; kk < BK / 32; kk++) mmaF8(d, smemDescSw128(aAddr + kk * 32), smemDescSw128(bAddr + kk * 32), idesc, kk != 0);
          }
          mmaCommit(&done[stage]);  // the stage is free and the group's products are complete once these MMAs are
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    const int q = warp & 3;         // the quarter of tensor-memory lanes this warp may read
    const int h = (warp - 2) >> 2;  // which of the two warps of that quarter: columns [32h, 32h+32) and [64+32h, 64+32h+32)
    int stage = 0;
    uint32_t phase = 0, grp = 0;
    bool ok = true;
    for (int t = cta; t < numTiles && ok; t += nctas) {
      int tm, tn;
      pol.coord(t, p.tilesM, p.tilesN, tm, tn);
      if (!pol.valid(tm, tn)) continue;
      if (!pol.epiBegin(tm, err)) { ok = false; break; }
      const int row = tm * BM + q * 32 + lane;
      const float* sB = p.sB + (size_t)pol.scaleBOff(tm, tn);
      float acc[kAccCols];
#pragma unroll
      for (int i = 0; i < kAccCols; i++) acc[i] = 0.f;
      for (int g = 0; g < kGroups; g++) {
        const uint32_t ab = grp % kAccGroups;
        grp++;
        float s[kGroup];
#pragma unroll
        for (int j = 0; j < kGroup; j++) {
          const int kb = g * kGroup + j;
          s[j] = (row < p.M && kb < p.kBlocks) ? pol.scaleA(kb, row) * __ldg(sB + kb) : 0.f;
        }
        if (!mbarWait(&done[stage], phase, err, gemm::ERR_EPI_ACC_FULL)) { ok = false; break; }
        if (++stage == kStages) { stage = 0; phase ^= 1; }
        tcFenceAfter();
#pragma unroll
        for (int j = 0; j < kGroup; j++) {
          const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (ab * kGroup + j) * BN + h * 32;
          uint32_t x0[32], x1[32];
          tmemLoad32(taddr, x0);
          tmemLoad32(taddr + 64, x1);
          tmemLoadWait();
#pragma unroll
          for (int i = 0; i < 32; i++) {
            acc[i] = fmaf(s[j], __uint_as_float(x0[i]), acc[i]);
            acc[32 + i] = fmaf(s[j], __uint_as_float(x1[i]), acc[32 + i]);
          }
        }
        tcFenceBefore();
        __syncwarp();
        if (lane == 0) mbarArrive(&partEmpty[ab]);
      }
      if (!ok) break;
      pol.emit(acc, tm, tn, q, h, lane, epiStage + (size_t)(warp - 2) * kEpiBytesPerWarp);
      pol.tileDone(tm, tn, q, h, lane);
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
  __device__ __forceinline__ void emit(float (&acc)[kAccCols], int tm, int tn, int q, int h, int lane, uint8_t* sw) const {
    const int row0 = tm * BM + q * 32;
    storeCols<64>(
        sw, lane, p.N - tn * BN, acc,
        [&](int r) -> __nv_bfloat16* { return row0 + r < p.M ? p.C + (size_t)(row0 + r) * p.ldc + (size_t)tn * BN : nullptr; },
        [&](int g) { return g * 64 + h * 32; });
  }
  __device__ __forceinline__ void tileDone(int, int, int, int, int) const {}
};

}  // namespace gemm8
}  // namespace b200
