// Persistent, warp-specialised bf16 GEMM on the 5th-generation tensor cores:
//   C[M, N] = A[M, K] * B[N, K]^T   (both operands K-major, as in y = x W^T)
// A CTA walks output tiles of 128 x BN. Warp 0 feeds shared memory with TMA tile loads through a
// ring of mbarrier-guarded stages, warp 1 issues tcgen05.mma from a single thread into a
// double-buffered fp32 accumulator in tensor memory, warps 2..5 drain finished accumulators with
// tcgen05.ld and run the epilogue, so the epilogue of tile t overlaps the main loop of tile t+1.
// Tile order, operand readiness and the epilogue are hooks of a policy object, which is where the
// fused GEMM+collective kernels differ from the plain GEMM.
// Every wait is bounded; on a failed wait the kernel records an error code, drains and returns.
#pragma once

#include "sm100.cuh"

namespace b200 {
namespace gemm {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int kThreads = 192;

template <int BN> struct Cfg {
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr uint32_t kABytes = BM * BK * 2;
  static constexpr uint32_t kBBytes = BN * BK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators of BN fp32 columns
  static constexpr uint32_t kEpiBytesPerWarp = 32 * 128 * 2;  // 32 rows x 128 bf16 columns staged per epilogue warp
  static constexpr size_t kSmemBytes =
      (size_t)kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + 4 * kEpiBytesPerWarp;
};

struct Params {
  CUtensorMap mapA;  // [M, K] bf16, box {BK, BM}, 128-byte swizzle
  CUtensorMap mapB;  // [N, K] bf16, box {BK, BN}, 128-byte swizzle
  int M, N, K;
  int tilesM, tilesN;
  int* err;          // device word: 0, or the code of the first wait that gave up
};

enum ErrCode : int { ERR_PRODUCER_EMPTY = 1, ERR_MMA_FULL = 2, ERR_MMA_ACC_EMPTY = 3, ERR_EPI_ACC_FULL = 4, ERR_FLAG_WAIT = 5, ERR_REDUCE_WAIT = 6 };

// Default tile order: walk M fastest inside bands of `kBand` N-tiles so that concurrently running
// CTAs share B tiles (and, across a band, A tiles) in L2.
__device__ __forceinline__ void bandedCoord(int t, int tilesM, int tilesN, int& tm, int& tn) {
  constexpr int kBand = 8;
  const int perBand = kBand * tilesM;
  const int band = t / perBand;
  const int inBand = t - band * perBand;
  const int bandW = min(kBand, tilesN - band * kBand);
  tn = band * kBand + inBand % bandW;
  tm = inBand / bandW;
}

// fp32 accumulator words -> bf16, 32 consecutive columns of one row, to global memory.
__device__ __forceinline__ void storeRow32Bf16(__nv_bfloat16* dst, const uint32_t (&acc)[32], int validCols) {
  if (validCols >= 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
    for (int v = 0; v < 4; v++) {
      uint4 o;
      uint32_t* ow = &o.x;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(acc[v * 8 + 2 * i]), __uint_as_float(acc[v * 8 + 2 * i + 1]));
        ow[i] = *reinterpret_cast<uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(dst + v * 8) = o;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; i++)
      if (i < validCols) dst[i] = __float2bfloat16(__uint_as_float(acc[i]));
  }
}

// Epilogue through shared memory, so that global (or peer) stores are whole 256-byte row segments
// instead of 64 bytes per thread. A warp owns 32 accumulator rows. For every group of 128 output
// columns: each lane converts its row's 4 x 32 columns to bf16 and parks them in the warp's
// staging buffer (16-byte chunks XOR-swizzled by the row so neither phase has bank conflicts);
// then half-warps walk the rows and write 256 contiguous bytes each.
//   loadChunk(c, acc)  fills acc[32] (fp32 bit patterns) with output columns [32c, 32c+32) of the lane's row
//   rowPtr(r)          destination of output column 0 of the warp's r-th row, or nullptr to skip the row
//   outCols            output columns of this tile (multiple of 32); colLimit: how many of them exist
template <typename LoadChunk, typename RowPtr>
__device__ __forceinline__ void drainStaged(uint8_t* sw, int lane, int outCols, int colLimit, LoadChunk loadChunk, RowPtr rowPtr) {
  for (int h = 0; h * 128 < outCols; h++) {
    const int colsHere = min(128, outCols - h * 128);
    const int chunks32 = colsHere / 32;
#pragma unroll 1
    for (int c = 0; c < chunks32; c++) {
      uint32_t acc[32];
      loadChunk(h * 4 + c, acc);
#pragma unroll
      for (int v = 0; v < 4; v++) {
        uint4 o;
        uint32_t* ow = &o.x;
#pragma unroll
        for (int i = 0; i < 4; i++) {
          __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(acc[v * 8 + 2 * i]), __uint_as_float(acc[v * 8 + 2 * i + 1]));
          ow[i] = *reinterpret_cast<uint32_t*>(&hh);
        }
        const int j = c * 4 + v;  // 16-byte chunk inside the 256-byte staged row
        *reinterpret_cast<uint4*>(sw + lane * 256 + ((j ^ (lane & 7)) << 4)) = o;
      }
    }
    __syncwarp();
    const int chunksRow = colsHere / 8;       // 16-byte chunks per staged row (16 for a full group)
    const int sub = lane & 15, half = lane >> 4;
    const int validChunks = max(0, min(chunksRow, (colLimit - h * 128) / 8));
#pragma unroll 1
    for (int r2 = 0; r2 < 32; r2 += 2) {
      const int r = r2 + half;
      __nv_bfloat16* dst = rowPtr(r);
      if (dst != nullptr && sub < validChunks) {
        const uint4 v = *reinterpret_cast<const uint4*>(sw + r * 256 + ((sub ^ (r & 7)) << 4));
        *reinterpret_cast<uint4*>(dst + h * 128 + sub * 8) = v;
      }
    }
    // Ragged right edge (fewer than 8 columns left in a chunk): element by element.
    const int tailStart = h * 128 + validChunks * 8;
    const int tailEnd = min(colLimit, h * 128 + colsHere);
    if (tailStart < tailEnd) {
      __nv_bfloat16* dst = rowPtr(lane);
      if (dst != nullptr)
        for (int col = tailStart; col < tailEnd; col++) {
          const int jj = (col - h * 128) >> 3;
          dst[col] = reinterpret_cast<const __nv_bfloat16*>(sw + lane * 256 + ((jj ^ (lane & 7)) << 4))[col & 7];
        }
    }
    __syncwarp();
  }
}

// Policy interface (all __device__):
//   void coord(int t, int tilesM, int tilesN, int& tm, int& tn)        tile order
//   bool valid(int tm, int tn)                                         false: the tile is skipped by every role
//   int aRow(int tm), int bRow(int tm, int tn)                         first row of the tile in the A / B tensor maps
//   bool waitTile(int tm, int tn, volatile int* err)                   producer: operands of the tile are in place
//   void drain(uint32_t taddr, int tm, int tn, int q, int lane, uint8_t* sw)  epilogue warp q: read its 32 accumulator rows at taddr (+column)
//                                                                      and emit them (sw: the warp's 8 KiB staging buffer)
//   void tileDone(int tm, int tn, int q, int lane)                     epilogue thread, after its rows of the tile are out
template <int BN, typename Policy>
__device__ __forceinline__ void gemmCta(const Params& p, Policy& pol, int cta, int nctas, uint8_t* smemRaw) {
  using C = Cfg<BN>;
  using namespace sm100;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smemA = smem;
  uint8_t* smemB = smem + (size_t)C::kStages * C::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)C::kStages * C::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::kStages;
  uint64_t* accFull = bars + 2 * C::kStages;
  uint64_t* accEmpty = accFull + 2;
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(accEmpty + 2);
  uint8_t* epiStage = reinterpret_cast<uint8_t*>(bars) + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* err = p.err;

  if (threadIdx.x == 0) {
    prefetchTensorMap(&p.mapA);
    prefetchTensorMap(&p.mapB);
    for (int s = 0; s < C::kStages; s++) {
      mbarInit(&full[s], 1);
      mbarInit(&empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbarInit(&accFull[b], 1);
      mbarInit(&accEmpty[b], 4);  // one arrival per epilogue warp
    }
    fenceBarrierInit();
  }
  if (warp == 1) {
    tmemAlloc(tmemSlot, C::kTmemCols);
    tmemRelinquish();
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmem = *tmemSlot;

  const int numTiles = p.tilesM * p.tilesN;
  const int kIters = (p.K + BK - 1) / BK;

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
        const int aRow = pol.aRow(tm), bRow = pol.bRow(tm, tn);
        for (int k = 0; k < kIters; k++) {
          if (!mbarWait(&empty[stage], phase ^ 1, err, ERR_PRODUCER_EMPTY)) { ok = false; break; }
          mbarArriveExpectTx(&full[stage], C::kStageBytes);
          tmaLoad2d(smemA + (size_t)stage * C::kABytes, &p.mapA, k * BK, aRow, &full[stage]);
          tmaLoad2d(smemB + (size_t)stage * C::kBBytes, &p.mapB, k * BK, bRow, &full[stage]);
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Let loads already in flight land before the CTA goes away.
        for (int s = 0; s < C::kStages; s++) mbarWait(&full[s], 0, err, 0, 2000u);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instrDesc(BM, BN, 1 /*bf16*/);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = cta; t < numTiles && ok; t += nctas) {
        {
          int tm, tn;
          pol.coord(t, p.tilesM, p.tilesN, tm, tn);
          if (!pol.valid(tm, tn)) continue;
        }
        const int b = it & 1;
        const uint32_t accPhase = (it >> 1) & 1;
        it++;
        if (!mbarWait(&accEmpty[b], accPhase ^ 1, err, ERR_MMA_ACC_EMPTY)) { ok = false; break; }
        tcFenceAfter();
        const uint32_t d = tmem + (uint32_t)b * BN;
        for (int k = 0; k < kIters; k++) {
          if (!mbarWait(&full[stage], phase, err, ERR_MMA_FULL)) { ok = false; break; }
          tcFenceAfter();
          const uint32_t aAddr = smemAddr(smemA + (size_t)stage * C::kABytes);
          const uint32_t bAddr = smemAddr(smemB + (size_t)stage * C::kBBytes);
#pragma unroll
          for (int kk = 0; kk < BK / 16; kk++)
            mmaF16(d, smemDescSw128(aAddr + kk * 32), smemDescSw128(bAddr + kk * 32), idesc, (k | kk) != 0);
          mmaCommit(&empty[stage]);  // the stage is free once these MMAs have read it
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) mmaCommit(&accFull[b]);
      }
    }
  } else {
    const int q = warp & 3;  // the quarter of tensor-memory lanes this warp may read
    int it = 0;
    bool ok = true;
    for (int t = cta; t < numTiles && ok; t += nctas) {
      int tm, tn;
      pol.coord(t, p.tilesM, p.tilesN, tm, tn);
      if (!pol.valid(tm, tn)) continue;
      const int b = it & 1;
      const uint32_t accPhase = (it >> 1) & 1;
      it++;
      if (!mbarWait(&accFull[b], accPhase, err, ERR_EPI_ACC_FULL)) { ok = false; break; }
      tcFenceAfter();
      pol.drain(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * BN), tm, tn, q, lane, epiStage + (size_t)q * C::kEpiBytesPerWarp);
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArrive(&accEmpty[b]);
      pol.tileDone(tm, tn, q, lane);
    }
  }
  tcFenceBefore();
  __syncthreads();
  if (warp == 1) tmemDealloc(tmem, C::kTmemCols);
}

// ---- the plain GEMM: banded order, nothing to wait for, C = bf16(acc) ------------------------------------
template <int BN> struct PlainPolicy {
  __nv_bfloat16* C;
  int ldc;
  int N;
  __device__ __forceinline__ void coord(int t, int tilesM, int tilesN, int& tm, int& tn) const { bandedCoord(t, tilesM, tilesN, tm, tn); }
  __device__ __forceinline__ bool valid(int, int) const { return true; }
  __device__ __forceinline__ int aRow(int tm) const { return tm * BM; }
  __device__ __forceinline__ int bRow(int, int tn) const { return tn * BN; }
  __device__ __forceinline__ bool waitTile(int, int, volatile int*) const { return true; }
  __device__ __forceinline__ void tileDone(int, int, int, int) const {}
  int M;
  __device__ __forceinline__ void drain(uint32_t taddr, int tm, int tn, int q, int lane, uint8_t* sw) const {
    const int row0 = tm * BM + q * 32;
    drainStaged(
        sw, lane, BN, N - tn * BN,
        [&](int c, uint32_t(&acc)[32]) {
          sm100::tmemLoad32(taddr + c * 32, acc);
          sm100::tmemLoadWait();
        },
        [&](int r) -> __nv_bfloat16* { return row0 + r < M ? C + (size_t)(row0 + r) * ldc + (size_t)tn * BN : nullptr; });
  }
};

template <int BN, typename Policy>
__global__ void __launch_bounds__(kThreads, 1) gemmKernel(const __grid_constant__ Params p, Policy pol) {
  extern __shared__ uint8_t smemRaw[];
  gemmCta<BN>(p, pol, blockIdx.x, gridDim.x, smemRaw);
}

}  // namespace gemm
}  // namespace b200
