// Pieces shared by the bf16 and the fp8 forms of the fused tensor-parallel kernels (tp_fused.cu, tp_fused_fp8.cu):
// the peer pull of the all-gather side, and the staging layout, tile counters and reducer of the reduce-scatter side.
#pragma once

#include "../coll/prims.cuh"
#include "../core/comm.h"
#include "gemm_sm100.cuh"

namespace b200 {
namespace tp {

using gemm::BM;

__device__ __forceinline__ void pullBlock(char* dst, const char* src, size_t bytes) {
  // 16 independent 16-byte loads per thread in flight: peer loads are latency bound.
  const int t = threadIdx.x, nt = blockDim.x;
  const size_t nvec = bytes >> 4;
  const uint4* s = (const uint4*)src;
  uint4* d = (uint4*)dst;
  size_t i = t;
  constexpr int U = 16;
  for (; i + (size_t)(U - 1) * nt < nvec; i += (size_t)U * nt) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; u++) v[u] = ldStream16(s + i + (size_t)u * nt);
#pragma unroll
    for (int u = 0; u < U; u++) st16(d + i + (size_t)u * nt, v[u]);
  }
  for (; i < nvec; i += nt) st16(d + i, ldStream16(s + i));
}

struct RsArgs {
  char* stagePeer[kMaxRanks];   // every rank's staging window as mapped here
  size_t stageOff;              // byte offset of this call's parity half inside the window
  size_t flagOff;               // byte offset of this call's parity counters inside the window
  uint32_t target;              // counter value that means "all n partials of the tile are here"
  int rowsPerRank, blocksPerRank;
  int N;                        // columns of the output
  __nv_bfloat16* y;             // [rowsPerRank, N] owned rows of the result
  int ldy;
};

// Epilogue side of a finished partial tile: once all epilogue warps (`epiThreads` threads) have stored their part, one
// thread (`leader`) bumps the tile's counter at the owner. tileW: columns per tile (the counters are indexed in tiles of
// that width).
__device__ __forceinline__ void rsTileDone(const RsArgs& a, int tileW, int tm, int tn, bool leader, int epiThreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(epiThreads) : "memory");
  if (leader) {
    const int owner = tm / a.blocksPerRank;
    const int tilesN = (a.N + tileW - 1) / tileW;
    uint32_t* f = (uint32_t*)(a.stagePeer[owner] + a.flagOff) + (size_t)(tm - owner * a.blocksPerRank) * tilesN + tn;
    __threadfence_system();
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(f) : "memory");
  }
}

// Reducer phase, run by every CTA after its GEMM tiles: sum the n staged partials of every tile this rank owns.
template <int BN>
__device__ __forceinline__ void reduceOwnedTiles(const RsArgs& a, int rank, int n, int* errWord) {
  __shared__ int ok;
  const int tilesN = (a.N + BN - 1) / BN;
  const int owned = a.blocksPerRank * tilesN;
  const char* stage = a.stagePeer[rank] + a.stageOff;
  const uint32_t* flags = (const uint32_t*)(a.stagePeer[rank] + a.flagOff);
  const size_t slot = (size_t)a.rowsPerRank * a.N;  // elements per source rank
  for (int idx = blockIdx.x; idx < owned; idx += gridDim.x) {
    if (threadIdx.x == 0) {
      int good = 0;
      for (uint32_t i = 0; i < 200000000u; i++) {
        if ((int32_t)(ldAcquireSys(flags + idx) - a.target) >= 0) { good = 1; break; }
        if ((i & 0x3ff) == 0x3ff && *(volatile int*)errWord) break;
        __nanosleep(32);
      }
      if (!good) atomicCAS(errWord, 0, gemm::ERR_REDUCE_WAIT);
      ok = good;
    }
    __syncthreads();
    if (ok) {
      const int tmL = idx / tilesN, tn = idx % tilesN;
      const int cols = min(BN, a.N - tn * BN);
      const int vecPerRow = cols >> 3;
      for (int v = threadIdx.x; v < BM * vecPerRow; v += blockDim.x) {
        const int r = v / vecPerRow, cv = v - r * vecPerRow;
        const int row = tmL * BM + r;
        if (row >= a.rowsPerRank) continue;
        const size_t e = (size_t)row * a.N + (size_t)tn * BN + (size_t)cv * 8;
        float acc[8];
#pragma unroll
        for (int s = 0; s < kMaxRanks; s++) {
          if (s < n) {
            const uint4 x = ldStream16(stage + (s * slot + e) * 2);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
            for (int k = 0; k < 4; k++) {
              const float2 f = __bfloat1622float2(h[k]);
              acc[2 * k] = s == 0 ? f.x : acc[2 * k] + f.x;
              acc[2 * k + 1] = s == 0 ? f.y : acc[2 * k + 1] + f.y;
            }
          }
        }
        uint4 o;
        uint32_t* ow = &o.x;
#pragma unroll
        for (int k = 0; k < 4; k++) {
          __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
          ow[k] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(a.y + (size_t)row * a.ldy + (size_t)tn * BN + (size_t)cv * 8) = o;
      }
    }
    __syncthreads();
  }
}

// ---- host side -----------------------------------------------------------------------------------------------------
bool peersOf(Comm* c, const void* p, size_t bytes, char* (&out)[kMaxRanks]);
// Flags of the all-gather side (one word per block of 128 rows, local device memory, grown on demand) and the sequence
// number of this call on the communicator.
ncclResult_t agNextCall(Comm* c, int needFlags, uint32_t** flags, uint32_t* seq);
// Number of earlier reduce-scatter calls on (communicator, workspace); the workspace is bound to the tile width of its
// first call, because the tile counters are laid out by it.
ncclResult_t rsNextCall(Comm* c, const void* workspace, int tileW, unsigned long long* calls);

struct DevGuard2 {
  int prev = -1, want;
  explicit DevGuard2(int d) : want(d) { cudaGetDevice(&prev); if (prev != want) cudaSetDevice(want); }
  ~DevGuard2() { if (prev != want && prev >= 0) cudaSetDevice(prev); }
};

template <typename K>
cudaError_t allowSmem(K kernel, size_t bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace tp
}  // namespace b200
