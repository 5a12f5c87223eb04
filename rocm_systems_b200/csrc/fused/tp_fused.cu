// Tensor-parallel hot paths as ONE kernel each: the collective runs inside the tcgen05 GEMM.
//
//   all-gather -> GEMM (+SwiGLU)   X is row-sharded over the ranks. A few "communication" CTAs pull
//       the peers' shards over NVLink (plain peer loads) into this GPU's copy of X, 128 rows at a
//       time, and publish a flag per block of rows; the GEMM CTAs start on the local shard and take
//       the remote row blocks in the order they land, their TMA producer waiting on the flag of
//       the block it needs. The remote tile crosses NVLink once, lands in local memory, and is read
//       from there by ordinary (non-multicast) TMA loads.
//   GEMM -> reduce-scatter         every rank multiplies its K-shard; the epilogue converts each
//       accumulator tile to bf16 and stores it straight into the staging buffer of the rank that
//       owns those rows (peer stores), tiles of remote owners first, then bumps a per-tile counter
//       at the owner. When a CTA runs out of GEMM tiles it turns reducer: it waits for a tile's
//       counter to reach the rank count, adds the n partials in fp32 and writes the owned rows.
// No barrier between the ranks is needed on the GEMM->RS path: staging and counters are double
// buffered by call parity and counters only grow. Every wait is bounded.
#include <map>
#include <mutex>

#include <algorithm>

#include "../core/cudrv.h"
#include "b200coll/fused.h"
#include "gemm_host.h"
#include "tp_fused.cuh"

namespace b200 {
namespace tp {

using namespace gemm;

// ---- all-gather -> GEMM ---------------------------------------------------------------------------------
struct AgArgs {
  char* xLocal;                 // this rank's copy of X: [n * rowsPerRank, K] bf16
  const char* xPeer[kMaxRanks]; // the peers' copies (their own shard is valid there)
  uint32_t* flags;              // local device memory: [n * blocksPerRank], last sequence number landed
  uint32_t seq;                 // sequence number of this call
  int rowsPerRank, blocksPerRank;  // blocks of BM rows
  size_t rowBytes;              // K * 2
  int nComm;                    // communication CTAs (the first blocks of the grid)
  __nv_bfloat16* out;           // [M, Nout]
  int ldo, nOut;
};

template <int BN, bool SWIGLU> struct AgPolicy {
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
  __device__ __forceinline__ int aRow(int tm) const { return tm * BM; }
  __device__ __forceinline__ int bRow(int, int tn) const { return tn * BN; }
  __device__ __forceinline__ bool waitTile(int tm, int, volatile int* err) const {
    if (tm / a.blocksPerRank == rank) return true;
    const uint32_t* f = a.flags + tm;
    for (uint32_t i = 0; i < 200000000u; i++) {
      uint32_t v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if ((int32_t)(v - a.seq) >= 0) {
        asm volatile("fence.proxy.async;" ::: "memory");  // the TMA reads that follow see the pulled rows
        return true;
      }
      if ((i & 0x3ff) == 0x3ff && *err) return false;
      __nanosleep(32);
    }
    atomicCAS((int*)err, 0, ERR_FLAG_WAIT);
    return false;
  }
  __device__ __forceinline__ void tileDone(int, int, int, int) const {}
  __device__ __forceinline__ void drain(uint32_t taddr, int tm, int tn, int q, int lane, uint8_t* sw) const {
    const int row0 = tm * BM + q * 32;
    if constexpr (SWIGLU) {
      // The weight rows are interleaved per tile: BN/2 gate rows then BN/2 up rows, so one tile
      // holds both halves of BN/2 outputs.
      drainStaged(
          sw, lane, BN / 2, a.nOut - tn * (BN / 2),
          [&](int c, uint32_t(&g)[32]) {
            uint32_t u[32];
            sm100::tmemLoad32(taddr + c * 32, g);
            sm100::tmemLoad32(taddr + BN / 2 + c * 32, u);
            sm100::tmemLoadWait();
#pragma unroll
            for (int i = 0; i < 32; i++) {
              const float gv = __uint_as_float(g[i]);
              g[i] = __float_as_uint(gv / (1.f + __expf(-gv)) * __uint_as_float(u[i]));
            }
          },
          [&](int r) -> __nv_bfloat16* { return a.out + (size_t)(row0 + r) * a.ldo + (size_t)tn * (BN / 2); });
    } else {
      drainStaged(
          sw, lane, BN, a.nOut - tn * BN,
          [&](int c, uint32_t(&acc)[32]) {
            sm100::tmemLoad32(taddr + c * 32, acc);
            sm100::tmemLoadWait();
          },
          [&](int r) -> __nv_bfloat16* { return a.out + (size_t)(row0 + r) * a.ldo + (size_t)tn * BN; });
    }
  }
};

template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1) agGemmKernel(const __grid_constant__ Params p, const __grid_constant__ AgArgs a, const __grid_constant__ DevComm c) {
  extern __shared__ uint8_t smemRaw[];
  if ((int)blockIdx.x < a.nComm) {
    const int j = blockIdx.x, n = c.nranks, rank = c.rank;
    uint32_t epoch = c.local->barEpoch[j];
    ctaBarrier(c, epoch);  // every rank's own shard is in place
    const int total = (n - 1) * a.blocksPerRank;
    const size_t blockBytes = (size_t)BM * a.rowBytes;
    for (int id = j; id < total; id += a.nComm) {
      const int peer = (rank + 1 + id / a.blocksPerRank) % n;
      const int blk = peer * a.blocksPerRank + id % a.blocksPerRank;
      pullBlock(a.xLocal + (size_t)blk * blockBytes, a.xPeer[peer] + (size_t)blk * blockBytes, blockBytes);
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
  AgPolicy<BN, SWIGLU> pol{a, c.rank, c.nranks};
  gemmCta<BN>(p, pol, blockIdx.x - a.nComm, gridDim.x - a.nComm, smemRaw);
}

// ---- GEMM -> reduce-scatter --------------------------------------------------------------------------------
template <int BN> struct RsPolicy {
  RsArgs a;
  int rank, n;
  __device__ __forceinline__ void coord(int t, int, int tilesN, int& tm, int& tn) const {
    // Tiles of remote owners first (rank+1, rank+2, ...), the rows this rank owns last.
    const int perGroup = a.blocksPerRank * tilesN;
    const int g = t / perGroup, r = t - g * perGroup;
    const int owner = (rank + 1 + g) % n;
    tm = owner * a.blocksPerRank + r / tilesN;
    tn = r % tilesN;
  }
  __device__ __forceinline__ bool valid(int, int) const { return true; }
  __device__ __forceinline__ int aRow(int tm) const { return tm * BM; }
  __device__ __forceinline__ int bRow(int, int tn) const { return tn * BN; }
  __device__ __forceinline__ bool waitTile(int, int, volatile int*) const { return true; }
  __device__ __forceinline__ void drain(uint32_t taddr, int tm, int tn, int q, int lane, uint8_t* sw) const {
    const int owner = tm / a.blocksPerRank;
    const int localRow0 = tm * BM + q * 32 - owner * a.rowsPerRank;
    // Owner's staging: [src rank][rowsPerRank][N] bf16; whole 256-byte row pieces go over NVLink.
    __nv_bfloat16* base = (__nv_bfloat16*)(a.stagePeer[owner] + a.stageOff) + ((size_t)rank * a.rowsPerRank + localRow0) * a.N + (size_t)tn * BN;
    drainStaged(
        sw, lane, BN, a.N - tn * BN,
        [&](int c, uint32_t(&acc)[32]) {
          sm100::tmemLoad32(taddr + c * 32, acc);
          sm100::tmemLoadWait();
        },
        [&](int r) -> __nv_bfloat16* { return base + (size_t)r * a.N; });
  }
  __device__ __forceinline__ void tileDone(int tm, int tn, int q, int lane) const { rsTileDone(a, BN, tm, tn, q == 0 && lane == 0, 128); }
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1) gemmRsKernel(const __grid_constant__ Params p, const __grid_constant__ RsArgs a, const __grid_constant__ DevComm c) {
  extern __shared__ uint8_t smemRaw[];
  RsPolicy<BN> pol{a, c.rank, c.nranks};
  gemmCta<BN>(p, pol, blockIdx.x, gridDim.x, smemRaw);
  reduceOwnedTiles<BN>(a, c.rank, c.nranks, p.err);
}

}  // namespace tp
}  // namespace b200

// =================================================================================================
// Host entry points
// =================================================================================================
using namespace b200;
using namespace b200::tp;

namespace {

struct AgState {
  uint32_t* flags = nullptr; uint32_t seq = 0; int cap = 0;
  cudaStream_t side = nullptr;          // copy-engine mode: the stream of the pulls
  cudaEvent_t evStart = nullptr, evDone = nullptr;
};
struct RsState { unsigned long long calls = 0; int tileW = 0; };
std::mutex gTpMu;
std::map<Comm*, AgState> gAg;
std::map<std::pair<Comm*, const void*>, RsState> gRs;

// A freed workspace (or a communicator that goes away) takes its call counter along: the next workspace at that address
// starts at call 0, like its zeroed tile counters.
void tpForget(Comm* c, const void* base) {
  std::lock_guard<std::mutex> lk(gTpMu);
  for (auto it = gRs.begin(); it != gRs.end();) {
    if (it->first.first == c && (base == nullptr || it->first.second == base)) it = gRs.erase(it);
    else ++it;
  }
  if (base == nullptr) {
    auto it = gAg.find(c);
    if (it != gAg.end()) {
      if (it->second.flags) cudaFree(it->second.flags);
      if (it->second.side) cudaStreamDestroy(it->second.side);
      if (it->second.evStart) cudaEventDestroy(it->second.evStart);
      if (it->second.evDone) cudaEventDestroy(it->second.evDone);
      gAg.erase(it);
    }
  }
}

}  // namespace

namespace b200 {
namespace tp {

bool peersOf(Comm* c, const void* p, size_t bytes, char* (&out)[kMaxRanks]) {
  size_t off = 0;
  std::lock_guard<std::mutex> lk(c->mu);
  Window* w = c->findWindow(p, bytes, &off);
  if (!w) return false;
  for (int r = 0; r < c->nranks; r++) out[r] = w->seg.peer[r] + off;
  return true;
}

ncclResult_t agNextCall(Comm* c, int needFlags, uint32_t** flags, uint32_t* seq) {
  addReleaseNotifier(tpForget);
  std::lock_guard<std::mutex> lk(gTpMu);
  AgState& st = gAg[c];
  if (st.cap < needFlags) {
    if (st.flags) cudaFree(st.flags);
    st.flags = nullptr;
    st.cap = 0;
    BCUDA(cudaMalloc(&st.flags, (size_t)needFlags * 4));
    BCUDA(cudaMemset(st.flags, 0, (size_t)needFlags * 4));
    st.cap = needFlags;
    st.seq = 0;
  }
  *flags = st.flags;
  *seq = ++st.seq;
  return ncclSuccess;
}

// Copy-engine form of the all-gather side: the peers' shards are pulled by cudaMemcpyAsync on a side stream, a few row
// blocks per copy, in the order the GEMM takes them (rank + 1, rank + 2, ...); behind every copy a stream memory write
// publishes the flags of its row blocks. No SM pulls anything, so the GEMM keeps all of them. The side stream starts once
// `stream` has reached this call (this rank's own rows are written) and all ranks have met at a barrier; a second barrier
// behind the copies tells every rank that its shard is no longer being read, and `stream` joins the side stream behind the
// kernel the caller launches next. Flags and tile waits are the ones of the kernel's own communication CTAs.
ncclResult_t agPullByCopyEngine(Comm* c, ncclComm_t comm, char* xLocal, char* const* xPeer, uint32_t* flags, uint32_t seq, int blocksPerRank,
                                size_t blockBytes, cudaStream_t stream, cudaEvent_t* joinAfterKernel) {
  const CuDrv& d = CuDrv::get();
  if (!d.cuStreamWriteValue32) BFAIL(ncclInvalidUsage, "copy-engine all-gather needs stream memory operations (cuStreamWriteValue32), which this driver lacks");
  cudaStream_t side;
  cudaEvent_t evStart, evDone;
  {
    std::lock_guard<std::mutex> lk(gTpMu);
    AgState& st = gAg[c];
    if (!st.side) {
      BCUDA(cudaStreamCreateWithFlags(&st.side, cudaStreamNonBlocking));
      BCUDA(cudaEventCreateWithFlags(&st.evStart, cudaEventDisableTiming));
      BCUDA(cudaEventCreateWithFlags(&st.evDone, cudaEventDisableTiming));
    }
    side = st.side; evStart = st.evStart; evDone = st.evDone;
  }
  const int n = c->nranks, rank = c->rank;
  BCUDA(cudaEventRecord(evStart, stream));
  BCUDA(cudaStreamWaitEvent(side, evStart, 0));
  BCHECK(b200collBarrier(comm, side));  // every rank's own shard is in place
  const int group = blocksPerRank >= 4 ? blocksPerRank / 4 : 1;  // row blocks per copy: four copies per peer shard
  for (int i = 1; i < n; i++) {
    const int peer = (rank + i) % n;
    for (int b0 = 0; b0 < blocksPerRank; b0 += group) {
      const int nb = std::min(group, blocksPerRank - b0);
      const size_t off = (size_t)(peer * blocksPerRank + b0) * blockBytes;
      BCUDA(cudaMemcpyAsync(xLocal + off, xPeer[peer] + off, (size_t)nb * blockBytes, cudaMemcpyDeviceToDevice, side));
      for (int b = 0; b < nb; b++)
        BCU(d.cuStreamWriteValue32((CUstream)side, (CUdeviceptr)(flags + peer * blocksPerRank + b0 + b), seq, CU_STREAM_WRITE_VALUE_DEFAULT));
    }
  }
  BCHECK(b200collBarrier(comm, side));  // the peers are done reading this rank's shard
  BCUDA(cudaEventRecord(evDone, side));
  *joinAfterKernel = evDone;
  return ncclSuccess;
}

ncclResult_t rsNextCall(Comm* c, const void* workspace, int tileW, unsigned long long* calls) {
  addReleaseNotifier(tpForget);
  std::lock_guard<std::mutex> lk(gTpMu);
  RsState& st = gRs[std::make_pair(c, workspace)];
  if (st.tileW == 0) st.tileW = tileW;
  if (st.tileW != tileW)
    BFAIL(ncclInvalidUsage, "GEMM->reduce-scatter workspace %p was first used with %d-column tiles, this call needs %d: give each shape its own workspace",
          workspace, st.tileW, tileW);
  *calls = st.calls++;
  return ncclSuccess;
}

}  // namespace tp
}  // namespace b200

extern "C" {

size_t b200collGemmRsWorkspaceBytes(int rowsPerRank, int N, int nranks) {
  const size_t stage = (size_t)nranks * rowsPerRank * N * 2;
  const size_t flags = (((size_t)((rowsPerRank + 127) / 128) * ((N + 127) / 128) * 4) + 255) & ~(size_t)255;
  return 2 * stage + 2 * flags;
}

ncclResult_t b200collAgGemm(ncclComm_t comm, void* xSym, const void* w, void* out, int rowsPerRank, int wRows, int K, int swiglu, int commCtas,
                            cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  const int n = c->nranks;
  if (!xSym || !w || !out) BFAIL(ncclInvalidArgument, "b200collAgGemm: null buffer");
  if (rowsPerRank <= 0 || rowsPerRank % BM) BFAIL(ncclInvalidArgument, "b200collAgGemm: rows per rank (%d) must be a multiple of %d", rowsPerRank, BM);
  if (K % 8 || wRows % 128) BFAIL(ncclInvalidArgument, "b200collAgGemm: K %% 8 and weight rows %% 128 must be 0");
  const int bn = (wRows % 256 == 0) ? 256 : 128;
  const int M = rowsPerRank * n;
  if (c->asyncError.load() != ncclSuccess) BFAIL((ncclResult_t)c->asyncError.load(), "communicator is in an error state: %s", c->lastErr.c_str());
  DevGuard2 g(c->cudaDev);
  AgArgs a{};
  char* peers[kMaxRanks] = {};
  if (n > 1) {
    if (!peersOf(c, xSym, (size_t)M * K * 2, peers)) BFAIL(ncclInvalidUsage, "b200collAgGemm: X must live in symmetric memory (b200collSymAlloc)");
  } else {
    peers[0] = (char*)xSym;
  }
  for (int r = 0; r < n; r++) a.xPeer[r] = peers[r];
  a.xLocal = (char*)xSym;
  a.rowsPerRank = rowsPerRank;
  a.blocksPerRank = rowsPerRank / BM;
  a.rowBytes = (size_t)K * 2;
  // Who pulls the peers' rows: copy engines (commCtas < 0), that many CTAs (> 0), or the measured better of the two
  // (0): from four ranks up the copy engines, which leave every SM to the GEMM (8 GPUs, 8192 x 8192 x 7168: 0.83 ms
  // against 1.00 ms with 20 pulling CTAs; between two GPUs the two are level).
  const bool byCopyEngine = n > 1 && (commCtas < 0 || (commCtas == 0 && n >= 4 && CuDrv::get().cuStreamWriteValue32 != nullptr));
  a.nComm = (n > 1 && !byCopyEngine) ? (commCtas > 0 ? commCtas : 20) : 0;
  if (a.nComm > 64) a.nComm = 64;
  a.out = (__nv_bfloat16*)out;
  a.nOut = swiglu ? wRows / 2 : wRows;
  a.ldo = a.nOut;
  BCHECK(agNextCall(c, n * a.blocksPerRank, &a.flags, &a.seq));
  cudaEvent_t join = nullptr;
  if (byCopyEngine) BCHECK(agPullByCopyEngine(c, comm, a.xLocal, peers, a.flags, a.seq, a.blocksPerRank, (size_t)BM * a.rowBytes, stream, &join));
  Params p{};
  if (!makeTileMap(&p.mapA, xSym, M, K, K, BM, 2) || !makeTileMap(&p.mapB, w, wRows, K, K, bn, 2))
    BFAIL(ncclInvalidArgument, "b200collAgGemm: operands must be 16-byte aligned with rows a multiple of 16 bytes");
  p.M = M;
  p.N = wRows;
  p.K = K;
  p.tilesM = M / BM;
  p.tilesN = wRows / bn;
  p.err = errWord();
  if (!p.err) BFAIL(ncclUnhandledCudaError, "b200collAgGemm: no error word");
  DevComm dc = c->dev;
  dc.opSeq = ++c->opSeq;
  dc.stamp = nullptr;
  int gemmCtas = smCount() - a.nComm;
  if (gemmCtas > p.tilesM * p.tilesN) gemmCtas = p.tilesM * p.tilesN;
  const int grid = a.nComm + gemmCtas;
  cudaError_t e;
#define B200_AG_LAUNCH(BNV, SW)                                                              \
  do {                                                                                       \
    e = allowSmem(agGemmKernel<BNV, SW>, Cfg<BNV>::kSmemBytes);                               \
    if (e == cudaSuccess) {                                                                  \
      agGemmKernel<BNV, SW><<<grid, kThreads, Cfg<BNV>::kSmemBytes, stream>>>(p, a, dc);      \
      e = cudaGetLastError();                                                                \
    }                                                                                        \
  } while (0)
  if (bn == 256) { if (swiglu) B200_AG_LAUNCH(256, true); else B200_AG_LAUNCH(256, false); }
  else { if (swiglu) B200_AG_LAUNCH(128, true); else B200_AG_LAUNCH(128, false); }
#undef B200_AG_LAUNCH
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "b200collAgGemm launch failed: %s", cudaGetErrorString(e));
  if (join) BCUDA(cudaStreamWaitEvent(stream, join, 0));  // what follows on `stream` also follows the pulls and the closing barrier
  return ncclSuccess;
}

ncclResult_t b200collGemmRs(ncclComm_t comm, const void* a_, const void* w, void* workspaceSym, void* y, int rowsPerRank, int N, int K,
                            cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  const int n = c->nranks;
  if (!a_ || !w || !workspaceSym || !y) BFAIL(ncclInvalidArgument, "b200collGemmRs: null buffer");
  if (rowsPerRank <= 0 || rowsPerRank % BM) BFAIL(ncclInvalidArgument, "b200collGemmRs: rows per rank (%d) must be a multiple of %d", rowsPerRank, BM);
  if (K % 8 || N % 128) BFAIL(ncclInvalidArgument, "b200collGemmRs: K %% 8 and N %% 128 must be 0");
  const int bn = (N % 256 == 0) ? 256 : 128;
  const int M = rowsPerRank * n;
  if (c->asyncError.load() != ncclSuccess) BFAIL((ncclResult_t)c->asyncError.load(), "communicator is in an error state: %s", c->lastErr.c_str());
  DevGuard2 g(c->cudaDev);
  const size_t wsBytes = b200collGemmRsWorkspaceBytes(rowsPerRank, N, n);
  RsArgs a{};
  char* peers[kMaxRanks] = {};
  if (n > 1) {
    if (!peersOf(c, workspaceSym, wsBytes, peers)) BFAIL(ncclInvalidUsage, "b200collGemmRs: the workspace must be symmetric memory of b200collGemmRsWorkspaceBytes()");
  } else {
    peers[0] = (char*)workspaceSym;
  }
  for (int r = 0; r < n; r++) a.stagePeer[r] = peers[r];
  const size_t stage = (size_t)n * rowsPerRank * N * 2;
  const size_t flags = (wsBytes - 2 * stage) / 2;
  unsigned long long calls;
  BCHECK(rsNextCall(c, workspaceSym, bn, &calls));
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
  if (!makeTileMap(&p.mapA, a_, M, K, K, BM, 2) || !makeTileMap(&p.mapB, w, N, K, K, bn, 2))
    BFAIL(ncclInvalidArgument, "b200collGemmRs: operands must be 16-byte aligned with rows a multiple of 16 bytes");
  p.M = M;
  p.N = N;
  p.K = K;
  p.tilesM = M / BM;
  p.tilesN = N / bn;
  p.err = errWord();
  if (!p.err) BFAIL(ncclUnhandledCudaError, "b200collGemmRs: no error word");
  DevComm dc = c->dev;
  dc.opSeq = ++c->opSeq;
  dc.stamp = nullptr;
  int grid = smCount();
  if (grid > p.tilesM * p.tilesN) grid = p.tilesM * p.tilesN;
  cudaError_t e;
  if (bn == 256) {
    e = allowSmem(gemmRsKernel<256>, Cfg<256>::kSmemBytes);
    if (e == cudaSuccess) { gemmRsKernel<256><<<grid, kThreads, Cfg<256>::kSmemBytes, stream>>>(p, a, dc); e = cudaGetLastError(); }
  } else {
    e = allowSmem(gemmRsKernel<128>, Cfg<128>::kSmemBytes);
    if (e == cudaSuccess) { gemmRsKernel<128><<<grid, kThreads, Cfg<128>::kSmemBytes, stream>>>(p, a, dc); e = cudaGetLastError(); }
  }
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "b200collGemmRs launch failed: %s", cudaGetErrorString(e));
  return ncclSuccess;
}

}  // extern "C"
