// Persistent, warp-specialised bf16 GEMM on the 5th-generation tensor cores:
//   C[M, N] = A[M, K] * B[N, K]^T   (both operands K-major, as in y = x W^T)
// One CTA per SM walks output tiles of 128 x BN. Warp 0 feeds shared memory with TMA tile loads
// through a ring of mbarrier-guarded stages, warp 1 issues tcgen05.mma from a single thread into
// a double-buffered fp32 accumulator in tensor memory, warps 2..5 drain finished accumulators with
// tcgen05.ld and run the epilogue, so the epilogue of tile t overlaps the main loop of tile t+1.
// The epilogue is a template hook, which is where the fused GEMM+collective kernels differ.
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
  static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct Params {
  CUtensorMap mapA;  // [M, K] bf16, box {BK, BM}, 128-byte swizzle
  CUtensorMap mapB;  // [N, K] bf16, box {BK, BN}, 128-byte swizzle
  int M, N, K;
  int tilesM, tilesN;
  int* err;          // device word: 0, or the code of the first wait that gave up
};

enum ErrCode : int { ERR_PRODUCER_EMPTY = 1, ERR_MMA_FULL = 2, ERR_MMA_ACC_EMPTY = 3, ERR_EPI_ACC_FULL = 4, ERR_FLAG_WAIT = 5 };

// Tile order: walk M fastest inside bands of `kBand` N-tiles so that concurrently running CTAs
// share B tiles (and, across a band, A tiles) in L2.
__device__ __forceinline__ void tileCoord(int t, int tilesM, int tilesN, int& tm, int& tn) {
  constexpr int kBand = 8;
  const int perBand = kBand * tilesM;
  const int band = t / perBand;
  const int inBand = t - band * perBand;
  const int bandW = min(kBand, tilesN - band * kBand);
  tn = band * kBand + inBand % bandW;
  tm = inBand / bandW;
}

// Epilogue hook interface:
//   struct Epi { __device__ void tile(int tm, int tn, int row, int col0, const uint32_t (&acc)[32], bool rowOk) }
// called by each epilogue thread for its row and each group of 32 columns of the tile;
//   __device__ bool waitTile(int tm, int tn, volatile int* err)  lets the producer block until the operands of a tile are ready
//   __device__ void tileDone(int tm, int tn)                      called once per tile by one thread after all its rows are out.
template <int BN, typename Epi>
__global__ void __launch_bounds__(kThreads, 1) gemmKernel(const __grid_constant__ Params p, Epi epi) {
  using C = Cfg<BN>;
  using namespace sm100;
  extern __shared__ uint8_t smemRaw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smemA = smem;
  uint8_t* smemB = smem + (size_t)C::kStages * C::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)C::kStages * C::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::kStages;
  uint64_t* accFull = bars + 2 * C::kStages;
  uint64_t* accEmpty = accFull + 2;
  uint32_t* tmemSlot = reinterpret_cast<uint32_t*>(accEmpty + 2);

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
      for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x) {
        int tm, tn;
        tileCoord(t, p.tilesM, p.tilesN, tm, tn);
        if (!epi.waitTile(tm, tn, err)) { ok = false; break; }
        for (int k = 0; k < kIters; k++) {
          if (!mbarWait(&empty[stage], phase ^ 1, err, ERR_PRODUCER_EMPTY)) { ok = false; break; }
          mbarArriveExpectTx(&full[stage], C::kStageBytes);
          tmaLoad2d(smemA + (size_t)stage * C::kABytes, &p.mapA, k * BK, tm * BM, &full[stage]);
          tmaLoad2d(smemB + (size_t)stage * C::kBBytes, &p.mapB, k * BK, tn * BN, &full[stage]);
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
      for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x, it++) {
        const int b = it & 1;
        const uint32_t accPhase = (it >> 1) & 1;
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
    for (int t = blockIdx.x; t < numTiles && ok; t += gridDim.x, it++) {
      int tm, tn;
      tileCoord(t, p.tilesM, p.tilesN, tm, tn);
      const int b = it & 1;
      const uint32_t accPhase = (it >> 1) & 1;
      if (!mbarWait(&accFull[b], accPhase, err, ERR_EPI_ACC_FULL)) { ok = false; break; }
      tcFenceAfter();
      const int row = tm * BM + q * 32 + lane;
      const bool rowOk = row < p.M;
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        uint32_t acc[32];
        tmemLoad32(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * BN + c * 32), acc);
        tmemLoadWait();
        epi.tile(tm, tn, row, tn * BN + c * 32, acc, rowOk);
      }
      tcFenceBefore();
      __syncwarp();
      if (lane == 0) mbarArrive(&accEmpty[b]);
      epi.tileDone(tm, tn, warp == 2 && lane == 0, q);
    }
  }
  tcFenceBefore();
  __syncthreads();
  if (warp == 1) tmemDealloc(tmem, C::kTmemCols);
}

// ---- the plain epilogue: C = bf16(acc) --------------------------------------------------------------
struct EpiStoreBf16 {
  __nv_bfloat16* C;
  int ldc;
  int N;
  __device__ __forceinline__ bool waitTile(int, int, volatile int*) const { return true; }
  __device__ __forceinline__ void tileDone(int, int, bool, int) const {}
  __device__ __forceinline__ void tile(int, int, int row, int col0, const uint32_t (&acc)[32], bool rowOk) const {
    if (!rowOk || col0 >= N) return;
    __nv_bfloat16* dst = C + (size_t)row * ldc + col0;
    if (col0 + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
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
        if (col0 + i < N) dst[i] = __float2bfloat16(__uint_as_float(acc[i]));
    }
  }
};

}  // namespace gemm
}  // namespace b200
