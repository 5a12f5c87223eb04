// The two fused tensor-parallel kernels (tp_fused.cu) on block-scaled fp8 operands: the same overlap of NVLink traffic
// and tensor-core work, with the main loop of gemm_fp8_sm100.cuh.
//
//   all-gather -> GEMM (+SwiGLU)   X is quantised by its owner (e4m3 rows + one fp32 scale per row and 128 channels,
//       scales stored [K / 128][M]) and row-sharded over the ranks, so half the bytes of the bf16 form cross NVLink.
//       Communication CTAs pull a block of 128 rows AND its K / 128 x 128 scales from the owner, then publish the
//       block's flag; the TMA producer of a GEMM CTA waits for the flag before it loads the rows, and the epilogue
//       warps take the same flag (an acquire of their own) before they read the block's scales.
//   GEMM -> reduce-scatter         both K-shards are fp8; the promoted fp32 tile leaves as bf16 partials for the owner of
//       its rows, exactly as in the bf16 kernel, and the same reducer sums them.
// Tiles are 128 x 128 (one weight scale per tile and K block); SwiGLU weights are interleaved per 128 rows: 64 gate rows,
// then the 64 up rows of the same outputs. Every wait is bounded.
#include "b200coll/fused.h"
#include "gemm_fp8_sm100.cuh"
#include "gemm_host.h"
#include "tp_fused.cuh"

namespace b200 {
namespace tp8 {

using namespace gemm8;
using tp::RsArgs;

// ---- all-gather -> GEMM ---------------------------------------------------------------------------------
struct AgArgs {
  char* xLocal;                  // this rank's copy of X: [n * rowsPerRank, K] e4m3
  const char* xPeer[kMaxRanks];  // the peers' copies (their own shard is valid there)
  float* sLocal;                 // this rank's copy of the scales: [K / 128][n * rowsPerRank]
  const float* sPeer[kMaxRanks];
  uint32_t* flags;               // local device memory: [n * blocksPerRank], last sequence number landed
  uint32_t seq;
  int rowsPerRank, blocksPerRank;
  int M, kBlocks;
  size_t rowBytes;               // K
  int nComm;                     // communication CTAs (the first blocks of the grid)
  __nv_bfloat16* out;            // [M, nOut]
  int ldo, nOut;
};

__device__ __forceinline__ float ldScale(const float* p) {
  float v;
  asm volatile("ld.relaxed.gpu.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait until block `blk` of rows (and its scales) has landed in this call; false: gave up or another wait did.
__device__ __forceinline__ bool waitBlockFlag(const uint32_t* f, uint32_t seq, volatile int* err, bool asyncProxy) {
  for (uint32_t i = 0; i < 200000000u; i++) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if ((int32_t)(v - seq) >= 0) {
      if (asyncProxy) asm volatile("fence.proxy.async;" ::: "memory");  // the TMA reads that follow see the pulled rows
      return true;
    }
    if ((i & 0x3ff) == 0x3ff && *err) return false;
    __nanosleep(32);
  }
  atomicCAS((int*)err, 0, gemm::ERR_FLAG_WAIT);
  return false;
}

template <bool SWIGLU> struct AgPolicy {
  AgArgs a;
  int rank, n;
  __device__ __forceinline__ void coord(int t, int, int tilesN, int& tm, int& tn) const {
    // Row blocks in arrival order: the local shard, then peers rank+1, rank+2, ...
    const int perGroup = a.blocksPerRank * tilesN;
    const int g = t / perGroup, r = t - g * perGroup;
    const int owner = (rank + g) % n;
    tm = owner * a.blocksPerRank + r / tilesN;
    tn = r % tilesN;
  }
  __device__ __forceinline__ bool valid(int, int) const { return true; }
  __device__ __forceinline__ int bRow(int, int tn) const { return tn * BN; }
  __device__ __forceinline__ int scaleBOff(int, int tn) const { return tn * a.kBlocks; }
  __device__ __forceinline__ bool waitTile(int tm, int, volatile int* err) const {
    if (tm / a.blocksPerRank == rank) return true;
    return waitBlockFlag(a.flags + tm, a.seq, err, true);
  }
  __device__ __forceinline__ bool epiBegin(int tm, volatile int* err) const {
    if (tm / a.blocksPerRank == rank) return true;
    return waitBlockFlag(a.flags + tm, a.seq, err, false);
  }
  __device__ __forceinline__ float scaleA(int kb, int row) const { return ldScale(a.sLocal + (size_t)kb * a.M + row); }
  __device__ __forceinline__ void emit(float (&acc)[kAccCols], int tm, int tn, int q, int h, int lane, uint8_t* sw) const {
    const int row0 = tm * BM + q * 32;
    if constexpr (SWIGLU) {
      // The thread holds gate columns 32h .. 32h+32 of the tile in acc[0..32) and the up columns of the same outputs in acc[32..64).
#pragma unroll
      for (int i = 0; i < 32; i++) {
        const float g = acc[i];
        acc[i] = g / (1.f + __expf(-g)) * acc[32 + i];
      }
      storeCols<32>(
          sw, lane, a.nOut - tn * (BN / 2), acc, [&](int r) -> __nv_bfloat16* { return a.out + (size_t)(row0 + r) * a.ldo + (size_t)tn * (BN / 2); },
          [&](int) { return h * 32; });
    } else {
      storeCols<64>(
          sw, lane, a.nOut - tn * BN, acc, [&](int r) -> __nv_bfloat16* { return a.out + (size_t)(row0 + r) * a.ldo + (size_t)tn * BN; },
          [&](int g) { return g * 64 + h * 32; });
    }
  }
  __device__ __forceinline__ void tileDone(int, int, int, int, int) const {}
};

template <bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1) agGemmFp8Kernel(const __grid_constant__ Params p, const __grid_constant__ AgArgs a, const __grid_constant__ DevComm c) {
  extern __shared__ uint8_t smemRaw[];
  if ((int)blockIdx.x < a.nComm) {
    const int j = blockIdx.x, n = c.nranks, rank = c.rank;
    uint32_t epoch = c.local->barEpoch[j];
    ctaBarrier(c, epoch);  // every rank's own shard and scales are in place
    const int total = (n - 1) * a.blocksPerRank;
    const size_t blockBytes = (size_t)BM * a.rowBytes;
    for (int id = j; id < total; id += a.nComm) {
      const int peer = (rank + 1 + id / a.blocksPerRank) % n;
      const int blk = peer * a.blocksPerRank + id % a.blocksPerRank;
      tp::pullBlock(a.xLocal + (size_t)blk * blockBytes, a.xPeer[peer] + (size_t)blk * blockBytes, blockBytes);
      // The block's scales: 128 floats (32 x 16 bytes) out of every row of the [K / 128][M] table.
      for (int v = threadIdx.x; v < a.kBlocks * 32; v += blockDim.x) {
        const size_t e = (size_t)(v >> 5) * a.M + (size_t)blk * BM + (size_t)(v & 31) * 4;
        st16(reinterpret_cast<uint4*>(a.sLocal + e), ldStream16(reinterpret_cast<const uint4*>(a.sPeer[peer] + e)));
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence();
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a.flags + blk), "r"(a.seq) : "memory");
      }
    }
    ctaBarrier(c, epoch);  // the peers are done reading this rank's shard
    if (threadIdx.x == 0) c.local->barEpoch[j] = epoch;
    return;
  }
  AgPolicy<SWIGLU> pol{a, c.rank, c.nranks};
  gemmFp8Cta(p, pol, blockIdx.x - a.nComm, gridDim.x - a.nComm, smemRaw);
}

// ---- GEMM -> reduce-scatter --------------------------------------------------------------------------------
struct RsPolicy {
  const RsArgs& a;  // the kernel's __grid_constant__ parameter
  const float* sA;  // [K / 128][M], local
  int M, kBlocks, rank, n;
  __device__ __forceinline__ bool valid(int, int) const { return true; }
  __device__ __forceinline__ int bRow(int, int tn) const { return tn * BN; }
  __device__ __forceinline__ int scaleBOff(int, int tn) const { return tn * kBlocks; }
  __device__ __forceinline__ void coord(int t, int, int tilesN, int& tm, int& tn) const {
    // Tiles of remote owners first (rank+1, rank+2, ...), the rows this rank owns last.
    const int perGroup = a.blocksPerRank * tilesN;
    const int g = t / perGroup, r = t - g * perGroup;
    const int owner = (rank + 1 + g) % n;
    tm = owner * a.blocksPerRank + r / tilesN;
    tn = r % tilesN;
  }
  __device__ __forceinline__ bool waitTile(int, int, volatile int*) const { return true; }
  __device__ __forceinline__ bool epiBegin(int, volatile int*) const { return true; }
  __device__ __forceinline__ float scaleA(int kb, int row) const { return __ldg(sA + (size_t)kb * M + row); }
  __device__ __forceinline__ void emit(float (&acc)[kAccCols], int tm, int tn, int q, int h, int lane, uint8_t* sw) const {
    const int owner = tm / a.blocksPerRank;
    const int localRow0 = tm * BM + q * 32 - owner * a.rowsPerRank;
    // Owner's staging: [src rank][rowsPerRank][N] bf16; 64-byte row pieces go over NVLink.
    __nv_bfloat16* base = (__nv_bfloat16*)(a.stagePeer[owner] + a.stageOff) + ((size_t)rank * a.rowsPerRank + localRow0) * a.N + (size_t)tn * BN;
    storeCols<64>(
        sw, lane, a.N - tn * BN, acc, [&](int r) -> __nv_bfloat16* { return base + (size_t)r * a.N; }, [&](int g) { return g * 64 + h * 32; });
  }
  __device__ __forceinline__ void tileDone(int tm, int tn, int q, int h, int lane) const {
    tp::rsTileDone(a, BN, tm, tn, q == 0 && h == 0 && lane == 0, kEpiThreads);
  }
};

__global__ void __launch_bounds__(kThreads, 1) gemmRsFp8Kernel(const __grid_constant__ Params p, const __grid_constant__ RsArgs a, const __grid_constant__ DevComm c) {
  extern __shared__ uint8_t smemRaw[];
  RsPolicy pol{a, p.sA, p.M, p.kBlocks, c.rank, c.nranks};
  gemmFp8Cta(p, pol, blockIdx.x, gridDim.x, smemRaw);
  tp::reduceOwnedTiles<BN>(a, c.rank, c.nranks, p.err);
}

}  // namespace tp8
}  // namespace b200

// =================================================================================================
// Host entry points
// =================================================================================================
using namespace b200;
using namespace b200::tp8;

extern "C" {

ncclResult_t b200collAgGemmFp8(ncclComm_t comm, void* x8Sym, float* sASym, const void* w8, const float* sW, void* out, int rowsPerRank, int wRows, int K,
                               int swiglu, int commCtas, cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  const int n = c->nranks;
  if (!x8Sym || !sASym || !w8 || !sW || !out) BFAIL(ncclInvalidArgument, "b200collAgGemmFp8: null buffer");
  if (rowsPerRank <= 0 || rowsPerRank % BM) BFAIL(ncclInvalidArgument, "b200collAgGemmFp8: rows per rank (%d) must be a multiple of %d", rowsPerRank, BM);
  if (K <= 0 || K % 128 || wRows <= 0 || wRows % 128) BFAIL(ncclInvalidArgument, "b200collAgGemmFp8: K and weight rows must be positive multiples of 128");
  if (((uintptr_t)sASym & 15) || ((uintptr_t)out & 15)) BFAIL(ncclInvalidArgument, "b200collAgGemmFp8: scales and output must be 16-byte aligned");
  const int M = rowsPerRank * n;
  if (c->asyncError.load() != ncclSuccess) BFAIL((ncclResult_t)c->asyncError.load(), "communicator is in an error state: %s", c->lastErr.c_str());
  tp::DevGuard2 g(c->cudaDev);
  AgArgs a{};
  char* xp[kMaxRanks] = {};
  char* sp[kMaxRanks] = {};
  const int kBlocks = K / 128;
  if (n > 1) {
    if (!tp::peersOf(c, x8Sym, (size_t)M * K, xp) || !tp::peersOf(c, sASym, (size_t)kBlocks * M * 4, sp))
      BFAIL(ncclInvalidUsage, "b200collAgGemmFp8: X and its scales must live in symmetric memory (b200collSymAlloc)");
  } else {
    xp[0] = (char*)x8Sym;
    sp[0] = (char*)sASym;
  }
  for (int r = 0; r < n; r++) {
    a.xPeer[r] = xp[r];
    a.sPeer[r] = (const float*)sp[r];
  }
  a.xLocal = (char*)x8Sym;
  a.sLocal = sASym;
  a.rowsPerRank = rowsPerRank;
  a.blocksPerRank = rowsPerRank / BM;
  a.M = M;
  a.kBlocks = kBlocks;
  a.rowBytes = (size_t)K;
  a.nComm = n > 1 ? (commCtas > 0 ? commCtas : 16) : 0;
  if (a.nComm > 64) a.nComm = 64;
  a.out = (__nv_bfloat16*)out;
  a.nOut = swiglu ? wRows / 2 : wRows;
  a.ldo = a.nOut;
  BCHECK(tp::agNextCall(c, n * a.blocksPerRank, &a.flags, &a.seq));
  Params p{};
  if (!gemm::makeTileMap(&p.mapA, x8Sym, M, K, K, BM, 1) || !gemm::makeTileMap(&p.mapB, w8, wRows, K, K, BN, 1))
    BFAIL(ncclInvalidArgument, "b200collAgGemmFp8: operands must be 16-byte aligned");
  p.sA = sASym;
  p.sB = sW;
  p.C = a.out;
  p.M = M;
  p.N = wRows;
  p.K = K;
  p.ldc = a.ldo;
  p.tilesM = M / BM;
  p.tilesN = wRows / BN;
  p.kBlocks = kBlocks;
  p.err = gemm::errWord();
  if (!p.err) BFAIL(ncclUnhandledCudaError, "b200collAgGemmFp8: no error word");
  DevComm dc = c->dev;
  dc.opSeq = ++c->opSeq;
  dc.stamp = nullptr;
  int gemmCtas = gemm::smCount() - a.nComm;
  if (gemmCtas > p.tilesM * p.tilesN) gemmCtas = p.tilesM * p.tilesN;
  const int grid = a.nComm + gemmCtas;
  cudaError_t e;
  if (swiglu) {
    e = tp::allowSmem(agGemmFp8Kernel<true>, kSmemBytes);
    if (e == cudaSuccess) { agGemmFp8Kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(p, a, dc); e = cudaGetLastError(); }
  } else {
    e = tp::allowSmem(agGemmFp8Kernel<false>, kSmemBytes);
    if (e == cudaSuccess) { agGemmFp8Kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(p, a, dc); e = cudaGetLastError(); }
  }
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "b200collAgGemmFp8 launch failed: %s", cudaGetErrorString(e));
  return ncclSuccess;
}

ncclResult_t b200collGemmRsFp8(ncclComm_t comm, const void* a8, const float* sA, const void* w8, const float* sW, void* workspaceSym, void* y,
                               int rowsPerRank, int N, int K, cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  const int n = c->nranks;
  if (!a8 || !sA || !w8 || !sW || !workspaceSym || !y) BFAIL(ncclInvalidArgument, "b200collGemmRsFp8: null buffer");
  if (rowsPerRank <= 0 || rowsPerRank % BM) BFAIL(ncclInvalidArgument, "b200collGemmRsFp8: rows per rank (%d) must be a multiple of %d", rowsPerRank, BM);
  if (K <= 0 || K % 128 || N <= 0 || N % 128) BFAIL(ncclInvalidArgument, "b200collGemmRsFp8: K and N must be positive multiples of 128");
  if ((uintptr_t)y & 15) BFAIL(ncclInvalidArgument, "b200collGemmRsFp8: the output must be 16-byte aligned");
  const int M = rowsPerRank * n;
  if (c->asyncError.load() != ncclSuccess) BFAIL((ncclResult_t)c->asyncError.load(), "communicator is in an error state: %s", c->lastErr.c_str());
  tp::DevGuard2 g(c->cudaDev);
  const size_t wsBytes = b200collGemmRsWorkspaceBytes(rowsPerRank, N, n);
  RsArgs a{};
  char* peers[kMaxRanks] = {};
  if (n > 1) {
    if (!tp::peersOf(c, workspaceSym, wsBytes, peers))
      BFAIL(ncclInvalidUsage, "b200collGemmRsFp8: the workspace must be symmetric memory of b200collGemmRsWorkspaceBytes()");
  } else {
    peers[0] = (char*)workspaceSym;
  }
  for (int r = 0; r < n; r++) a.stagePeer[r] = peers[r];
  const size_t stage = (size_t)n * rowsPerRank * N * 2;
  const size_t flags = (wsBytes - 2 * stage) / 2;
  unsigned long long calls;
  BCHECK(tp::rsNextCall(c, workspaceSym, BN, &calls));
  const int parity = (int)(calls & 1);
  a.stageOff = (size_t)parity * stage;
  a.flagOff = 2 * stage + (size_t)parity * flags;
  a.target = (uint32_t)((calls / 2 + 1) * (unsigned long long)n);
  a.rowsPerRank = rowsPerRank;
  a.blocksPerRank = rowsPerRank / BM;
  a.N = N;
  a.y = (__nv_bfloat16*)y;
  a.ldy = N;
  Params p{};
  if (!gemm::makeTileMap(&p.mapA, a8, M, K, K, BM, 1) || !gemm::makeTileMap(&p.mapB, w8, N, K, K, BN, 1))
    BFAIL(ncclInvalidArgument, "b200collGemmRsFp8: operands must be 16-byte aligned");
  p.sA = sA;
  p.sB = sW;
  p.C = a.y;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = N;
  p.tilesM = M / BM;
  p.tilesN = N / BN;
  p.kBlocks = K / 128;
  p.err = gemm::errWord();
  if (!p.err) BFAIL(ncclUnhandledCudaError, "b200collGemmRsFp8: no error word");
  DevComm dc = c->dev;
  dc.opSeq = ++c->opSeq;
  dc.stamp = nullptr;
  int grid = gemm::smCount();
  if (grid > p.tilesM * p.tilesN) grid = p.tilesM * p.tilesN;
  cudaError_t e = tp::allowSmem(gemmRsFp8Kernel, kSmemBytes);
  if (e == cudaSuccess) {
    gemmRsFp8Kernel<<<grid, kThreads, kSmemBytes, stream>>>(p, a, dc);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "b200collGemmRsFp8 launch failed: %s", cudaGetErrorString(e));
  return ncclSuccess;
}

}  // extern "C"
