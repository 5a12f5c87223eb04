// Mixture-of-experts expert parallelism: routing, dispatch, grouped expert GEMMs and combine.
//
//   epRoute     top-k of the router logits and the softmax of the selected logits (one warp per token).
//   epDispatch  ONE kernel does route -> permute -> fp8 e4m3 quantise (one scale per 128 channels)
//               -> all-to-all: a warp quantises its token once, then for each of the token's k
//               experts reserves a row in that expert's receive buffer on the owning rank with a
//               remote atomic over NVLink and stores payload + scales there (device-initiated puts,
//               no host round trip, no count exchange). The last CTA tells every peer it is done;
//               CTA 0 waits (bounded) until every peer said so, so when the kernel ends the receive
//               buffers and the per-expert counts are complete.
//   epDequant   fp8 rows -> bf16 rows for the grouped GEMMs.
//   grouped GEMMs run on the tcgen05 kernel with a policy that walks a compact list of (expert, row block,
//               column block): only row blocks that hold tokens are numbered, so the persistent CTAs share the
//               real work evenly; the first one applies SwiGLU in its epilogue.
//   epCombine   ONE kernel at the token's home rank: for each of the k experts it pulls the expert's
//               output row from the owning rank (peer loads) and accumulates gate * row in fp32,
//               in the fixed order k = 0..k-1, so the result is deterministic.
// Receive buffers and counters are double buffered by call parity; counters of the other parity
// are cleared by the dispatch that does not use them.
#include <algorithm>
#include <map>
#include <mutex>

#include <cuda_fp8.h>

#include "../coll/prims.cuh"
#include "../core/comm.h"
#include "b200coll/fused.h"
#include "gemm_fp8_sm100.cuh"
#include "gemm_host.h"
#include "gemm_sm100.cuh"

namespace b200 {
namespace ep {

constexpr int kMaxTopK = 8;

// Layout of the symmetric EP window of one rank (all offsets in bytes, 256-byte aligned).
struct EpLayout {
  int nranks, expertsLocal, cap, hidden, ffn;
  size_t cntOff;      // uint32 cnt[2][expertsLocal]   rows reserved so far (per parity)
  size_t doneOff;     // uint32 done[2][kMaxRanks]     dispatch-complete marks from every source rank
  size_t payloadOff;  // uint8  [expertsLocal][cap][hidden]         fp8 e4m3
  size_t scaleOff;    // float  [expertsLocal][cap][hidden / 128]
  size_t metaOff;     // int2   [expertsLocal][cap]   (source rank, source token * 8 + k)
  size_t outOff;      // bf16   [expertsLocal][cap][hidden]          expert outputs (pulled by combine)
  size_t total;
};

__host__ inline EpLayout makeLayout(int nranks, int expertsLocal, int cap, int hidden, int ffn) {
  EpLayout L{};
  L.nranks = nranks; L.expertsLocal = expertsLocal; L.cap = cap; L.hidden = hidden; L.ffn = ffn;
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  size_t o = 0;
  L.cntOff = o; o = up(o + (size_t)2 * expertsLocal * 4);
  L.doneOff = o; o = up(o + (size_t)2 * kMaxRanks * 4);
  L.payloadOff = o; o = up(o + (size_t)expertsLocal * cap * hidden);
  L.scaleOff = o; o = up(o + (size_t)expertsLocal * cap * (hidden / 128) * 4);
  L.metaOff = o; o = up(o + (size_t)expertsLocal * cap * 8);
  L.outOff = o; o = up(o + (size_t)expertsLocal * cap * hidden * 2);
  L.total = o;
  return L;
}

// ---- routing ------------------------------------------------------------------------------------------
// logits [T, E] fp32; E <= 1024, multiple of 32. Writes expert ids (int32) and gate weights (fp32,
// softmax over the selected logits) for the top `k`, largest first; ties go to the lower expert id.
// A NaN logit counts as -inf and +inf as the largest finite value, so every id written lies in [0, E)
// and every weight is finite: a row with fewer than k selectable values (all NaN, mostly -inf) fills up
// with the lowest expert ids not yet taken, and a row whose selected logits are all -inf gets weights 1/k.
__global__ void __launch_bounds__(256) epRoute(const float* __restrict__ logits, int* __restrict__ topIdx, float* __restrict__ topW, int T, int E, int k) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* row = logits + (size_t)warp * E;
  const int per = E / 32;  // <= 32
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; i++) {
    float x = i < per ? row[i * 32 + lane] : -INFINITY;
    x = x == x ? fminf(x, 3.402823466e38f) : -INFINITY;
    v[i] = x;
  }
  uint32_t taken = 0;  // bit i: this lane's candidate i was selected in an earlier round
  float sel[kMaxTopK];
  int selIdx[kMaxTopK];
  for (int r = 0; r < k; r++) {
    float best = -INFINITY;
    int bi = 0x7fffffff;  // no candidate on this lane (all taken)
#pragma unroll
    for (int i = 0; i < 32; i++)
      if (i < per && !((taken >> i) & 1u) && (bi == 0x7fffffff || v[i] > best)) { best = v[i]; bi = i * 32 + lane; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    sel[r] = best;
    selIdx[r] = bi;  // k <= E: some lane always had a candidate, so bi < E
    if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
  }
  if (lane == 0) {
    const float m = sel[0];
    float s = 0.f;
    const bool flat = m == -INFINITY;  // nothing selectable in the row: uniform weights
    for (int r = 0; r < k; r++) s += flat ? 1.f : __expf(sel[r] - m);
    for (int r = 0; r < k; r++) {
      topIdx[(size_t)warp * k + r] = selIdx[r];
      topW[(size_t)warp * k + r] = (flat ? 1.f : __expf(sel[r] - m)) / s;
    }
  }
}

// ---- dispatch -------------------------------------------------------------------------------------------
struct DispatchArgs {
  const __nv_bfloat16* x;   // [T, hidden]
  const int* topIdx;        // [T, k]
  int* sentSlot;            // [T, k] row reserved at the destination expert, or -1 when it was full
  int T, k;
  char* win[kMaxRanks];     // the EP window of every rank
  EpLayout L;
  int parity;
  uint32_t doneValue;       // value written into done[parity][rank] at every peer
  uint32_t* ticket;         // local: CTAs finished (for the last-CTA signal)
  int* dropped;             // local: rows that found their expert full
};

__global__ void __launch_bounds__(256) epDispatch(const __grid_constant__ DispatchArgs a, const __grid_constant__ DevComm c) {
  const int lane = threadIdx.x & 31;
  const int warpsPerCta = blockDim.x >> 5;
  const int gw = blockIdx.x * warpsPerCta + (threadIdx.x >> 5), nw = gridDim.x * warpsPerCta;
  const int H = a.L.hidden, groups = H / 128, rounds = H / 256;  // a round = 32 lanes x 8 channels
  const int rank = c.rank;

  // The counters of the other parity belong to the next call: clear them now.
  if (blockIdx.x == 0) {
    uint32_t* cnt = (uint32_t*)(a.win[rank] + a.L.cntOff) + (size_t)(a.parity ^ 1) * a.L.expertsLocal;
    for (int i = threadIdx.x; i < a.L.expertsLocal; i += blockDim.x) cnt[i] = 0;
  }

  for (int t = gw; t < a.T; t += nw) {
    // Quantise the token once: lane l holds channels (j * 32 + l) * 8 .. +8 for every round j.
    uint2 q[28];   // up to 7168 channels
    float sc[28];  // scale of the lane's group in round j (valid on every lane of the half-warp)
    const uint4* xr = reinterpret_cast<const uint4*>(a.x + (size_t)t * H);
#pragma unroll
    for (int j = 0; j < 28; j++) {
      if (j < rounds) {
        const uint4 raw = xr[j * 32 + lane];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float f[8];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const float2 p = __bfloat1622float2(h[i]);
          f[2 * i] = p.x; f[2 * i + 1] = p.y;
          amax = fmaxf(amax, fmaxf(fabsf(p.x), fabsf(p.y)));
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));  // 16 lanes = 128 channels
        const float scale = fmaxf(amax, 1e-10f) * (1.f / 448.f);
            sc[j] = scale;
        uint32_t w[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
          const __nv_fp8x4_e4m3 p4(make_float4(__fdiv_rn(f[4 * i], scale), __fdiv_rn(f[4 * i + 1], scale), __fdiv_rn(f[4 * i + 2], scale), __fdiv_rn(f[4 * i + 3], scale)));
          w[i] = *reinterpret_cast<const uint32_t*>(&p4);
        }
        q[j] = make_uint2(w[0], w[1]);
      }
    }
    for (int r = 0; r < a.k; r++) {
      const int e = a.topIdx[(size_t)t * a.k + r];
      if (e < 0 || e >= a.L.nranks * a.L.expertsLocal) {  // not an expert: counted like a row that found its expert full, no window touched
        if (lane == 0) {
          atomicAdd(a.dropped, 1);
          a.sentSlot[(size_t)t * a.k + r] = -1;
        }
        continue;
      }
      const int dst = e / a.L.expertsLocal, el = e - dst * a.L.expertsLocal;
      int slot = 0;
      if (lane == 0) {
        uint32_t* cnt = (uint32_t*)(a.win[dst] + a.L.cntOff) + (size_t)a.parity * a.L.expertsLocal + el;
        asm volatile("atom.relaxed.sys.global.add.u32 %0, [%1], 1;" : "=r"(slot) : "l"(cnt) : "memory");
        if (slot >= a.L.cap) { slot = -1; atomicAdd(a.dropped, 1); }
        a.sentSlot[(size_t)t * a.k + r] = slot;
      }
      slot = __shfl_sync(0xffffffffu, slot, 0);
      if (slot < 0) continue;
      const size_t rowIdx = (size_t)el * a.L.cap + slot;
      uint2* pay = reinterpret_cast<uint2*>(a.win[dst] + a.L.payloadOff + rowIdx * H);
      float* scl = reinterpret_cast<float*>(a.win[dst] + a.L.scaleOff) + rowIdx * groups;
#pragma unroll
      for (int j = 0; j < 28; j++) {
        if (j < rounds) {
          pay[j * 32 + lane] = q[j];
          if ((lane & 15) == 0) scl[j * 2 + (lane >> 4)] = sc[j];
        }
      }
      if (lane == 0) reinterpret_cast<int2*>(a.win[dst] + a.L.metaOff)[rowIdx] = make_int2(rank, t * kMaxTopK + r);
    }
  }

  // Last CTA out tells every rank that this rank's rows have all been stored.
  __shared__ int last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    last = atomicAdd(a.ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last) {
    if (threadIdx.x < c.nranks) {
      __threadfence_system();
      uint32_t* f = (uint32_t*)(a.win[threadIdx.x] + a.L.doneOff) + (size_t)a.parity * kMaxRanks + rank;
      stReleaseSys(f, a.doneValue);
    }
    if (threadIdx.x == 0) *a.ticket = 0;
  }
  // CTA 0 holds the kernel open until every peer's rows are in.
  if (blockIdx.x == 0 && threadIdx.x < c.nranks) {
    const uint32_t* f = (const uint32_t*)(a.win[rank] + a.L.doneOff) + (size_t)a.parity * kMaxRanks + threadIdx.x;
    waitGe(c, f, a.doneValue, WAIT_FUSED, threadIdx.x);
  }
}

// ---- fp8 -> bf16 for the rows that arrived ------------------------------------------------------------------
__global__ void __launch_bounds__(256) epDequant(const char* __restrict__ win, EpLayout L, int parity, __nv_bfloat16* __restrict__ xb) {
  const int lane = threadIdx.x & 31;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = (gridDim.x * blockDim.x) >> 5;
  const uint32_t* cnt = (const uint32_t*)(win + L.cntOff) + (size_t)parity * L.expertsLocal;
  const int H = L.hidden, groups = H / 128, rounds = H / 256;
  const int totalRows = L.expertsLocal * L.cap;
  for (int rowIdx = gw; rowIdx < totalRows; rowIdx += nw) {
    const int e = rowIdx / L.cap, r = rowIdx - e * L.cap;
    const int have = min((int)cnt[e], L.cap);
    if (r >= have) continue;
    const uint2* pay = reinterpret_cast<const uint2*>(win + L.payloadOff + (size_t)rowIdx * H);
    const float* scl = reinterpret_cast<const float*>(win + L.scaleOff) + (size_t)rowIdx * groups;
    uint4* dst = reinterpret_cast<uint4*>(xb + (size_t)rowIdx * H);
    for (int j = 0; j < rounds; j++) {
      const uint2 q = pay[j * 32 + lane];
      const float s = scl[j * 2 + (lane >> 4)];
      const __nv_fp8x4_e4m3* p4 = reinterpret_cast<const __nv_fp8x4_e4m3*>(&q);
      const float4 lo = float4(p4[0]), hi = float4(p4[1]);
      uint4 o;
      __nv_bfloat162 h0 = __floats2bfloat162_rn(lo.x * s, lo.y * s), h1 = __floats2bfloat162_rn(lo.z * s, lo.w * s);
      __nv_bfloat162 h2 = __floats2bfloat162_rn(hi.x * s, hi.y * s), h3 = __floats2bfloat162_rn(hi.z * s, hi.w * s);
      o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
      o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
      dst[j * 32 + lane] = o;
    }
  }
}

// ---- grouped expert GEMM policy ------------------------------------------------------------------------------
using namespace gemm;
template <int BN, bool SWIGLU> struct GroupPolicy {
  const uint32_t* cnt;   // rows per expert (may exceed cap when rows were dropped)
  int experts;           // local experts
  const int* prefix;     // shared memory, filled by the kernel: row blocks with tokens before expert e; [experts] = all of them
  int cap, capTiles;     // rows reserved per expert, in rows and in BM-row blocks
  int wRows;             // weight rows per expert
  __nv_bfloat16* out;    // [expertsLocal * cap, nOut]
  int ldo, nOut;
  __device__ __forceinline__ int have(int e) const { return min((int)cnt[e], cap); }
  // Tile t of the COMPACT list: only row blocks that hold tokens are numbered, expert after expert, so every CTA of the
  // persistent grid gets the same share of real work however unevenly the tokens fell (a buffer is sized for several
  // times the average count, so most of its row blocks are empty). Indices past the end map to no tile.
  __device__ __forceinline__ void coord(int t, int, int tilesN, int& tm, int& tn) const {
    const int rb = t / tilesN;
    tn = t - rb * tilesN;
    tm = -1;
    if (rb >= prefix[experts]) return;
    int e = 0;
    while (prefix[e + 1] <= rb) e++;  // prefix[] sits in shared memory: a few cycles per step
    tm = e * capTiles + (rb - prefix[e]);
  }
  __device__ __forceinline__ bool valid(int tm, int) const { return tm >= 0; }
  __device__ __forceinline__ int aRow(int tm) const { return tm * BM; }
  __device__ __forceinline__ int bRow(int tm, int tn) const { return (tm / capTiles) * wRows + tn * BN; }
  __device__ __forceinline__ bool waitTile(int, int, volatile int*) const { return true; }
  __device__ __forceinline__ void tileDone(int, int, int, int) const {}
  __device__ __forceinline__ void drain(uint32_t taddr, int tm, int tn, int q, int lane, uint8_t* sw) const {
    const int e = tm / capTiles;
    const int row0 = tm * BM + q * 32;
    const int rowsHave = have(e) - (row0 - e * cap);  // rows of this warp's 32 that hold tokens
    if constexpr (SWIGLU) {
      drainStaged(
          sw, lane, BN / 2, nOut - tn * (BN / 2),
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
          [&](int r) -> __nv_bfloat16* { return r < rowsHave ? out + (size_t)(row0 + r) * ldo + (size_t)tn * (BN / 2) : nullptr; });
    } else {
      drainStaged(
          sw, lane, BN, nOut - tn * BN,
          [&](int c, uint32_t(&acc)[32]) {
            sm100::tmemLoad32(taddr + c * 32, acc);
            sm100::tmemLoadWait();
          },
          [&](int r) -> __nv_bfloat16* { return r < rowsHave ? out + (size_t)(row0 + r) * ldo + (size_t)tn * BN : nullptr; });
    }
  }
};

// ---- first expert GEMM straight on the received fp8 rows ---------------------------------------------------------
// The rows in the window already are what the block-scaled GEMM wants: e4m3 with one fp32 scale per row and 128
// channels (row-major here, [row][hidden / 128]). With the experts' gate/up weight quantised per 128 x 128 block
// (interleaved per 128 rows: 64 gate rows, then the 64 up rows of the same outputs) the dequantisation pass and its
// bf16 copy of the activations disappear, and the larger of the two GEMMs runs at fp8 rate.
struct GroupPolicy8 {
  const uint32_t* cnt;  // rows per expert (may exceed cap when rows were dropped)
  int experts;          // local experts
  const int* prefix;    // shared memory, filled by the kernel: row blocks with tokens before expert e; [experts] = all of them
  int cap, capTiles;
  int wRows;            // weight rows per expert (2 ffn)
  const float* sA;      // [expertsLocal * cap][groups]
  int groups;           // hidden / 128
  __nv_bfloat16* out;   // act [expertsLocal * cap, nOut]
  int ldo, nOut;
  __device__ __forceinline__ int have(int e) const { return min((int)cnt[e], cap); }
  // Tile t of the COMPACT list: only row blocks that hold tokens are numbered, expert after expert, so every CTA of the
  // persistent grid gets the same share of real work however unevenly the tokens fell (a buffer is sized for several
  // times the average count, so most of its row blocks are empty). Indices past the end map to no tile.
  __device__ __forceinline__ void coord(int t, int, int tilesN, int& tm, int& tn) const {
    const int rb = t / tilesN;
    tn = t - rb * tilesN;
    tm = -1;
    if (rb >= prefix[experts]) return;
    int e = 0;
    while (prefix[e + 1] <= rb) e++;  // prefix[] sits in shared memory: a few cycles per step
    tm = e * capTiles + (rb - prefix[e]);
  }
  __device__ __forceinline__ bool valid(int tm, int) const { return tm >= 0; }
  __device__ __forceinline__ int bRow(int tm, int tn) const { return (tm / capTiles) * wRows + tn * gemm8::BN; }
  __device__ __forceinline__ int scaleBOff(int tm, int tn) const { return ((tm / capTiles) * (wRows / gemm8::BN) + tn) * groups; }
  __device__ __forceinline__ bool waitTile(int, int, volatile int*) const { return true; }
  __device__ __forceinline__ bool epiBegin(int, volatile int*) const { return true; }
  __device__ __forceinline__ float scaleA(int kb, int row) const { return __ldg(sA + (size_t)row * groups + kb); }
  __device__ __forceinline__ void emit(float (&acc)[gemm8::kAccCols], int tm, int tn, int q, int h, int lane, uint8_t* sw) const {
    constexpr int H = gemm8::BN / 2;
    const int e = tm / capTiles;
    const int row0 = tm * gemm::BM + q * 32;
    const int rowsHave = have(e) - (row0 - e * cap);  // rows of this warp's 32 that hold tokens
    // gate columns 32h .. 32h+32 of the tile in acc[0..32), the up columns of the same outputs in acc[32..64)
#pragma unroll
    for (int i = 0; i < 32; i++) {
      const float g = acc[i];
      acc[i] = g / (1.f + __expf(-g)) * acc[32 + i];
    }
    gemm8::storeCols<32>(
        sw, lane, H, acc,  // ffn is a multiple of 128: every tile has all of its 64 output columns
        [&](int r) -> __nv_bfloat16* { return r < rowsHave ? out + (size_t)(row0 + r) * ldo + (size_t)tn * H : nullptr; }, [&](int) { return h * 32; });
  }
  __device__ __forceinline__ void tileDone(int, int, int, int, int) const {}
};

constexpr int kMaxLocalExperts = 64;

// Row blocks with tokens before every expert, once per CTA, into shared memory (the compact tile list of the policies).
__device__ __forceinline__ void fillBlockPrefix(int* prefix, const uint32_t* cnt, int experts, int cap) {
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < experts; e++) {
      prefix[e] = acc;
      acc += (min((int)cnt[e], cap) + gemm::BM - 1) / gemm::BM;
    }
    prefix[experts] = acc;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(gemm8::kThreads, 1) groupedGemmFp8Kernel(const __grid_constant__ gemm8::Params p, GroupPolicy8 pol) {
  extern __shared__ uint8_t smemRaw[];
  __shared__ int prefix[kMaxLocalExperts + 1];
  fillBlockPrefix(prefix, pol.cnt, pol.experts, pol.cap);
  pol.prefix = prefix;
  gemm8::gemmFp8Cta(p, pol, blockIdx.x, gridDim.x, smemRaw);
}

// ---- combine ---------------------------------------------------------------------------------------------------
struct CombineArgs {
  const int* topIdx;      // [T, k]
  const float* topW;      // [T, k]
  const int* sentSlot;    // [T, k]
  __nv_bfloat16* out;     // [T, hidden]
  int T, k;
  char* win[kMaxRanks];
  EpLayout L;
};

// A warp handles 1024 channels of one token: pulls the k expert rows and adds gate * row in fp32.
__global__ void __launch_bounds__(256) epCombine(const __grid_constant__ CombineArgs a) {
  const int lane = threadIdx.x & 31;
  const int H = a.L.hidden;
  const int chunks = H / 1024;  // tasks per token
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = (gridDim.x * blockDim.x) >> 5;
  for (int task = gw; task < a.T * chunks; task += nw) {
    const int t = task / chunks, ch = task - t * chunks;
    float acc[4][8];
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int i = 0; i < 8; i++) acc[j][i] = 0.f;
    for (int r0 = 0; r0 < a.k; r0 += 4) {
      uint4 v[4][4];
      float w[4];
#pragma unroll
      for (int rr = 0; rr < 4; rr++) {
        const int r = r0 + rr;
        w[rr] = 0.f;
        if (r < a.k) {
          const int slot = a.sentSlot[(size_t)t * a.k + r];
          const int e = a.topIdx[(size_t)t * a.k + r];
          if (slot >= 0 && slot < a.L.cap && e >= 0 && e < a.L.nranks * a.L.expertsLocal) {
            const int dst = e / a.L.expertsLocal, el = e - dst * a.L.expertsLocal;
            w[rr] = a.topW[(size_t)t * a.k + r];
            const uint4* src = reinterpret_cast<const uint4*>(a.win[dst] + a.L.outOff + ((size_t)el * a.L.cap + slot) * H * 2) + ch * 128;
#pragma unroll
            for (int j = 0; j < 4; j++) v[rr][j] = ldStream16(src + j * 32 + lane);
          }
        }
      }
#pragma unroll
      for (int rr = 0; rr < 4; rr++) {
        if (w[rr] != 0.f) {
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[rr][j]);
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const float2 f = __bfloat1622float2(h[i]);
              acc[j][2 * i] += w[rr] * f.x;
              acc[j][2 * i + 1] += w[rr] * f.y;
            }
          }
        }
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(a.out + (size_t)t * H) + ch * 128;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      uint4 o;
      uint32_t* ow = &o.x;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        __nv_bfloat162 h = __floats2bfloat162_rn(acc[j][2 * i], acc[j][2 * i + 1]);
        ow[i] = *reinterpret_cast<uint32_t*>(&h);
      }
      dst[j * 32 + lane] = o;
    }
  }
}

// ---- backward pass ---------------------------------------------------------------------------------------------
// The gradient of combine is a dispatch and the gradient of dispatch is a combine, over the SAME rows: a token's row keeps
// the slot it reserved in the forward pass (sentSlot at its home rank, meta at the expert's rank), so nothing is reserved
// again and no count is exchanged.
//   epGateGrad    home rank: d gate[t, r] = <dy[t], expert output row of (t, r)>, the row pulled from its owner as in combine.
//   epGatherGrad  expert's rank: for every row that arrived, pull dy of its token from the token's home rank and scale it
//                 by the token's gate weight there: the gradient with respect to the expert's output row.
// The expert GEMMs' gradients are grouped GEMMs on the transposed weights (b200collEpGroupedGemm); the input gradient is
// epCombine with unit weights over the rows the last grouped GEMM left in the window's output region.
struct GateGradArgs {
  const __nv_bfloat16* dy;  // [T, hidden]
  const int* topIdx;        // [T, k]
  const int* sentSlot;      // [T, k]
  float* dGate;             // [T, k]
  int T, k;
  char* win[kMaxRanks];
  EpLayout L;
};

__global__ void __launch_bounds__(256) epGateGrad(const __grid_constant__ GateGradArgs a) {
  const int lane = threadIdx.x & 31;
  const int H = a.L.hidden;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = (gridDim.x * blockDim.x) >> 5;
  for (int task = gw; task < a.T * a.k; task += nw) {
    const int t = task / a.k;
    const int slot = a.sentSlot[task], e = a.topIdx[task];
    float dot = 0.f;
    if (slot >= 0 && slot < a.L.cap && e >= 0 && e < a.L.nranks * a.L.expertsLocal) {
      const int dst = e / a.L.expertsLocal, el = e - dst * a.L.expertsLocal;
      const uint4* row = reinterpret_cast<const uint4*>(a.win[dst] + a.L.outOff + ((size_t)el * a.L.cap + slot) * H * 2);
      const uint4* g = reinterpret_cast<const uint4*>(a.dy + (size_t)t * H);
      for (int j = lane; j < H / 8; j += 32) {
        const uint4 rv = ldStream16(row + j), gv = g[j];
        const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&rv);
        const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const float2 x = __bfloat1622float2(rh[i]), y = __bfloat1622float2(gh[i]);
          dot += x.x * y.x + x.y * y.y;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) a.dGate[task] = dot;
  }
}

struct GatherGradArgs {
  const char* dyPeer[kMaxRanks];    // every rank's dy [T, hidden] bf16 (symmetric memory)
  const char* gatePeer[kMaxRanks];  // every rank's gate weights [T, k] fp32 (symmetric memory)
  const char* win;                  // this rank's window
  EpLayout L;
  int parity, k, T;
  __nv_bfloat16* dOut;              // [expertsLocal * cap, hidden]
};

__global__ void __launch_bounds__(256) epGatherGrad(const __grid_constant__ GatherGradArgs a) {
  const int lane = threadIdx.x & 31;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = (gridDim.x * blockDim.x) >> 5;
  const uint32_t* cnt = (const uint32_t*)(a.win + a.L.cntOff) + (size_t)a.parity * a.L.expertsLocal;
  const int2* meta = reinterpret_cast<const int2*>(a.win + a.L.metaOff);
  const int H = a.L.hidden;
  const int totalRows = a.L.expertsLocal * a.L.cap;
  for (int rowIdx = gw; rowIdx < totalRows; rowIdx += nw) {
    const int e = rowIdx / a.L.cap, r = rowIdx - e * a.L.cap;
    if (r >= min((int)cnt[e], a.L.cap)) continue;
    const int2 m = meta[rowIdx];
    const int src = m.x, t = m.y / kMaxTopK, kk = m.y - t * kMaxTopK;
    uint4* dst = reinterpret_cast<uint4*>(a.dOut + (size_t)rowIdx * H);
    if (src < 0 || src >= a.L.nranks || t < 0 || t >= a.T || kk >= a.k) {  // not a row of this pass: contributes nothing
      for (int j = lane; j < H / 8; j += 32) dst[j] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const float g = *reinterpret_cast<const float*>(a.gatePeer[src] + ((size_t)t * a.k + kk) * 4);
    const uint4* row = reinterpret_cast<const uint4*>(a.dyPeer[src] + (size_t)t * H * 2);
    for (int j = lane; j < H / 8; j += 32) {
      uint4 v = ldStream16(row + j);
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(h[i]);
        h[i] = __floats2bfloat162_rn(g * f.x, g * f.y);
      }
      dst[j] = v;
    }
  }
}

template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(gemm::kThreads, 1) groupedGemmKernel(const __grid_constant__ gemm::Params p, GroupPolicy<BN, SWIGLU> pol) {
  extern __shared__ uint8_t smemRaw[];
  __shared__ int prefix[kMaxLocalExperts + 1];
  fillBlockPrefix(prefix, pol.cnt, pol.experts, pol.cap);
  pol.prefix = prefix;
  gemm::gemmCta<BN>(p, pol, blockIdx.x, gridDim.x, smemRaw);
}

}  // namespace ep
}  // namespace b200

// =================================================================================================
// Host entry points
// =================================================================================================
using namespace b200;
using namespace b200::ep;

namespace {

struct EpState {
  unsigned long long calls = 0;   // dispatches so far on this window
  uint32_t* ticket = nullptr;     // device: CTA ticket + dropped-row counter
};
std::mutex gEpMu;
std::map<std::pair<Comm*, const void*>, EpState> gEp;

// A freed window (or a communicator that goes away) takes its call counter along: the next window at that address starts at call 0,
// like its zeroed counters.
void epForget(Comm* c, const void* base) {
  std::lock_guard<std::mutex> lk(gEpMu);
  for (auto it = gEp.begin(); it != gEp.end();) {
    if (it->first.first == c && (base == nullptr || it->first.second == base)) {
      if (it->second.ticket) cudaFree(it->second.ticket);
      it = gEp.erase(it);
    } else {
      ++it;
    }
  }
}

bool epPeers(Comm* c, const void* p, size_t bytes, char* (&out)[kMaxRanks]) {
  if (c->nranks == 1) { out[0] = (char*)p; return true; }
  size_t off = 0;
  std::lock_guard<std::mutex> lk(c->mu);
  Window* w = c->findWindow(p, bytes, &off);
  if (!w) return false;
  for (int r = 0; r < c->nranks; r++) out[r] = w->seg.peer[r] + off;
  return true;
}

struct EpGuard {
  int prev = -1, want;
  explicit EpGuard(int d) : want(d) { cudaGetDevice(&prev); if (prev != want) cudaSetDevice(want); }
  ~EpGuard() { if (prev != want && prev >= 0) cudaSetDevice(prev); }
};

ncclResult_t checkShape(int expertsLocal, int cap, int hidden, int ffn, int k) {
  if (expertsLocal > kMaxLocalExperts) BFAIL(ncclInvalidArgument, "EP: at most %d experts per rank", kMaxLocalExperts);
  if (expertsLocal <= 0 || cap <= 0 || cap % 128) BFAIL(ncclInvalidArgument, "EP: capacity per expert (%d) must be a positive multiple of 128", cap);
  if (hidden % 1024 || hidden > 7168) BFAIL(ncclInvalidArgument, "EP: hidden (%d) must be a multiple of 1024, at most 7168", hidden);
  if (ffn % 128) BFAIL(ncclInvalidArgument, "EP: expert FFN width (%d) must be a multiple of 128", ffn);
  if (k < 1 || k > kMaxTopK) BFAIL(ncclInvalidArgument, "EP: top-k must be in [1, %d]", kMaxTopK);
  return ncclSuccess;
}

template <int BN, bool SW>
cudaError_t launchGrouped(const gemm::Params& p, const GroupPolicy<BN, SW>& pol, cudaStream_t s) {
  cudaError_t e = cudaFuncSetAttribute(groupedGemmKernel<BN, SW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm::Cfg<BN>::kSmemBytes);
  if (e != cudaSuccess) return e;
  int grid = gemm::smCount();
  if (grid > p.tilesM * p.tilesN) grid = p.tilesM * p.tilesN;
  groupedGemmKernel<BN, SW><<<grid, gemm::kThreads, gemm::Cfg<BN>::kSmemBytes, s>>>(p, pol);
  return cudaGetLastError();
}

}  // namespace

extern "C" {

size_t b200collEpWorkspaceBytes(int nranks, int expertsLocal, int cap, int hidden, int ffn) {
  return makeLayout(nranks, expertsLocal, cap, hidden, ffn).total;
}

ncclResult_t b200collEpRoute(const float* logits, int* topIdx, float* topW, int T, int E, int k, cudaStream_t stream) {
  if (!logits || !topIdx || !topW) BFAIL(ncclInvalidArgument, "b200collEpRoute: null buffer");
  if (E % 32 || E > 1024 || k < 1 || k > kMaxTopK || k > E) BFAIL(ncclInvalidArgument, "b200collEpRoute: E must be a multiple of 32 up to 1024, k in [1, 8]");
  if (T == 0) return ncclSuccess;
  epRoute<<<(T + 7) / 8, 256, 0, stream>>>(logits, topIdx, topW, T, E, k);
  BCUDA(cudaGetLastError());
  return ncclSuccess;
}

ncclResult_t b200collEpDispatch(ncclComm_t comm, void* winSym, const void* xBf16, const int* topIdx, int* sentSlot, int T, int k, int expertsLocal,
                                int cap, int hidden, int ffn, cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  BCHECK(checkShape(expertsLocal, cap, hidden, ffn, k));
  if (!winSym || !xBf16 || !topIdx || !sentSlot) BFAIL(ncclInvalidArgument, "b200collEpDispatch: null buffer");
  if (c->asyncError.load() != ncclSuccess) BFAIL((ncclResult_t)c->asyncError.load(), "communicator is in an error state: %s", c->lastErr.c_str());
  EpGuard g(c->cudaDev);
  DispatchArgs a{};
  a.L = makeLayout(c->nranks, expertsLocal, cap, hidden, ffn);
  if (!epPeers(c, winSym, a.L.total, a.win)) BFAIL(ncclInvalidUsage, "b200collEpDispatch: the window must be symmetric memory of b200collEpWorkspaceBytes()");
  addReleaseNotifier(epForget);
  {
    std::lock_guard<std::mutex> lk(gEpMu);
    EpState& st = gEp[std::make_pair(c, (const void*)winSym)];
    if (!st.ticket) {
      BCUDA(cudaMalloc(&st.ticket, 64));
      BCUDA(cudaMemset(st.ticket, 0, 64));
    }
    a.parity = (int)(st.calls & 1);
    a.doneValue = (uint32_t)(st.calls / 2 + 1);
    st.calls++;
    a.ticket = st.ticket;
    a.dropped = (int*)(st.ticket + 4);
  }
  a.x = (const __nv_bfloat16*)xBf16;
  a.topIdx = topIdx;
  a.sentSlot = sentSlot;
  a.T = T;
  a.k = k;
  DevComm dc = c->dev;
  dc.opSeq = ++c->opSeq;
  dc.stamp = nullptr;
  int ctas = std::max(1, std::min((T + 7) / 8, 4 * gemm::smCount()));
  epDispatch<<<ctas, 256, 0, stream>>>(a, dc);
  BCUDA(cudaGetLastError());
  return ncclSuccess;
}

// Both grouped expert GEMMs on what arrived; results land in the window's output region. act [expertsLocal * cap, ffn] is
// scratch. bf16 form: the rows are dequantised into xb [expertsLocal * cap, hidden] first. fp8 form (w13Scales != nullptr):
// the first GEMM reads the window's e4m3 rows and scales in place against a block-quantised w13.
static ncclResult_t epExperts(const char* what, ncclComm_t comm, void* winSym, const void* w13, const float* w13Scales, const void* w2, void* xb, void* act,
                              int expertsLocal, int cap, int hidden, int ffn, cudaStream_t stream) {
  const bool fp8 = w13Scales != nullptr;
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  BCHECK(checkShape(expertsLocal, cap, hidden, ffn, 1));
  if (!winSym || !w13 || !w2 || (!fp8 && !xb) || !act) BFAIL(ncclInvalidArgument, "%s: null buffer", what);
  EpGuard g(c->cudaDev);
  const EpLayout L = makeLayout(c->nranks, expertsLocal, cap, hidden, ffn);
  int parity;
  {
    std::lock_guard<std::mutex> lk(gEpMu);
    auto it = gEp.find(std::make_pair(c, (const void*)winSym));
    if (it == gEp.end() || it->second.calls == 0) BFAIL(ncclInvalidUsage, "%s: no dispatch has run on this window", what);
    parity = (int)((it->second.calls - 1) & 1);
  }
  const char* win = (const char*)winSym;
  const uint32_t* cnt = (const uint32_t*)(win + L.cntOff) + (size_t)parity * expertsLocal;
  const int rows = expertsLocal * cap;
  const int wRows = 2 * ffn;
  if (fp8) {
    // GEMM 1: act = swiglu(dequant(rows) * dequant(w13)^T) on the window's payload.
    gemm8::Params p{};
    if (!gemm::makeTileMap(&p.mapA, win + L.payloadOff, rows, hidden, hidden, gemm::BM, 1) ||
        !gemm::makeTileMap(&p.mapB, w13, (uint64_t)expertsLocal * wRows, hidden, hidden, gemm8::BN, 1))
      BFAIL(ncclInvalidArgument, "%s: misaligned operands", what);
    p.sA = (const float*)(win + L.scaleOff);
    p.sB = w13Scales;
    p.C = (__nv_bfloat16*)act;
    p.M = rows; p.N = wRows; p.K = hidden; p.ldc = ffn;
    p.tilesM = rows / gemm::BM; p.tilesN = wRows / gemm8::BN; p.kBlocks = hidden / 128;
    p.err = gemm::errWord();
    if (!p.err) BFAIL(ncclUnhandledCudaError, "%s: no error word", what);
    GroupPolicy8 pol{cnt, expertsLocal, nullptr, cap, cap / gemm::BM, wRows, p.sA, hidden / 128, (__nv_bfloat16*)act, ffn, ffn};
    cudaError_t e = cudaFuncSetAttribute(groupedGemmFp8Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm8::kSmemBytes);
    if (e == cudaSuccess) {
      int grid = gemm::smCount();
      if (grid > p.tilesM * p.tilesN) grid = p.tilesM * p.tilesN;
      groupedGemmFp8Kernel<<<grid, gemm8::kThreads, gemm8::kSmemBytes, stream>>>(p, pol);
      e = cudaGetLastError();
    }
    if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "%s: first grouped GEMM failed to launch: %s", what, cudaGetErrorString(e));
  } else {
    epDequant<<<4 * gemm::smCount(), 256, 0, stream>>>(win, L, parity, (__nv_bfloat16*)xb);
    BCUDA(cudaGetLastError());
    // GEMM 1: act = swiglu(xb * w13^T), w13 [expertsLocal * 2 ffn, hidden] with gate/up interleaved per tile.
    const int bn = wRows % 256 == 0 ? 256 : 128;
    gemm::Params p{};
    if (!gemm::makeTileMap(&p.mapA, xb, rows, hidden, hidden, gemm::BM, 2) || !gemm::makeTileMap(&p.mapB, w13, (uint64_t)expertsLocal * wRows, hidden, hidden, bn, 2))
      BFAIL(ncclInvalidArgument, "%s: misaligned operands", what);
    p.M = rows; p.N = wRows; p.K = hidden; p.tilesM = rows / gemm::BM; p.tilesN = wRows / bn; p.err = gemm::errWord();
    cudaError_t e;
    if (bn == 256) e = launchGrouped(p, GroupPolicy<256, true>{cnt, expertsLocal, nullptr, cap, cap / gemm::BM, wRows, (__nv_bfloat16*)act, ffn, ffn}, stream);
    else e = launchGrouped(p, GroupPolicy<128, true>{cnt, expertsLocal, nullptr, cap, cap / gemm::BM, wRows, (__nv_bfloat16*)act, ffn, ffn}, stream);
    if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "%s: first grouped GEMM failed to launch: %s", what, cudaGetErrorString(e));
  }
  // GEMM 2: out = act * w2^T, w2 [expertsLocal * hidden, ffn].
  {
    const int bn = hidden % 256 == 0 ? 256 : 128;
    gemm::Params p{};
    __nv_bfloat16* out = (__nv_bfloat16*)((char*)winSym + L.outOff);
    if (!gemm::makeTileMap(&p.mapA, act, rows, ffn, ffn, gemm::BM, 2) || !gemm::makeTileMap(&p.mapB, w2, (uint64_t)expertsLocal * hidden, ffn, ffn, bn, 2))
      BFAIL(ncclInvalidArgument, "%s: misaligned operands", what);
    p.M = rows; p.N = hidden; p.K = ffn; p.tilesM = rows / gemm::BM; p.tilesN = hidden / bn; p.err = gemm::errWord();
    cudaError_t e;
    if (bn == 256) e = launchGrouped(p, GroupPolicy<256, false>{cnt, expertsLocal, nullptr, cap, cap / gemm::BM, hidden, out, hidden, hidden}, stream);
    else e = launchGrouped(p, GroupPolicy<128, false>{cnt, expertsLocal, nullptr, cap, cap / gemm::BM, hidden, out, hidden, hidden}, stream);
    if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "%s: second grouped GEMM failed to launch: %s", what, cudaGetErrorString(e));
  }
  return ncclSuccess;
}

ncclResult_t b200collEpExperts(ncclComm_t comm, void* winSym, const void* w13, const void* w2, void* xb, void* act, int expertsLocal, int cap,
                               int hidden, int ffn, cudaStream_t stream) {
  return epExperts("b200collEpExperts", comm, winSym, w13, nullptr, w2, xb, act, expertsLocal, cap, hidden, ffn, stream);
}

ncclResult_t b200collEpExpertsFp8(ncclComm_t comm, void* winSym, const void* w13Fp8, const float* w13Scales, const void* w2, void* act, int expertsLocal,
                                  int cap, int hidden, int ffn, cudaStream_t stream) {
  if (!w13Scales) BFAIL(ncclInvalidArgument, "b200collEpExpertsFp8: null weight scales");
  return epExperts("b200collEpExpertsFp8", comm, winSym, w13Fp8, w13Scales, w2, nullptr, act, expertsLocal, cap, hidden, ffn, stream);
}

ncclResult_t b200collEpCombine(ncclComm_t comm, void* winSym, const int* topIdx, const float* topW, const int* sentSlot, void* out, int T, int k,
                               int expertsLocal, int cap, int hidden, int ffn, cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  BCHECK(checkShape(expertsLocal, cap, hidden, ffn, k));
  if (!winSym || !topIdx || !topW || !sentSlot || !out) BFAIL(ncclInvalidArgument, "b200collEpCombine: null buffer");
  EpGuard g(c->cudaDev);
  CombineArgs a{};
  a.L = makeLayout(c->nranks, expertsLocal, cap, hidden, ffn);
  if (!epPeers(c, winSym, a.L.total, a.win)) BFAIL(ncclInvalidUsage, "b200collEpCombine: the window must be symmetric memory");
  a.topIdx = topIdx; a.topW = topW; a.sentSlot = sentSlot; a.out = (__nv_bfloat16*)out; a.T = T; a.k = k;
  if (c->nranks > 1) BCHECK(b200collBarrier(comm, stream));  // every rank's expert outputs are written
  const int tasks = T * (hidden / 1024);
  int ctas = std::max(1, std::min((tasks + 7) / 8, 8 * gemm::smCount()));
  epCombine<<<ctas, 256, 0, stream>>>(a);
  BCUDA(cudaGetLastError());
  return ncclSuccess;
}

// ---- backward pass ---------------------------------------------------------------------------------------------
static ncclResult_t epLatestParity(const char* what, Comm* c, const void* winSym, int* parity) {
  std::lock_guard<std::mutex> lk(gEpMu);
  auto it = gEp.find(std::make_pair(c, winSym));
  if (it == gEp.end() || it->second.calls == 0) BFAIL(ncclInvalidUsage, "%s: no dispatch has run on this window", what);
  *parity = (int)((it->second.calls - 1) & 1);
  return ncclSuccess;
}

// out[rows of expert e] = a[rows of expert e] * w[e]^T for every local expert, over the rows of the latest dispatch:
// a [expertsLocal * cap, K], w [expertsLocal * wRows, K], out [expertsLocal * cap, wRows] (nullptr: the window's output
// region, which needs wRows == hidden). Row blocks without tokens are skipped. The three GEMMs of the experts' backward
// pass (and the recomputation of the gate/up pre-activations) are calls of this with transposed weights.
ncclResult_t b200collEpGroupedGemm(ncclComm_t comm, void* winSym, const void* a, const void* w, void* out, int wRows, int K, int expertsLocal, int cap,
                                   int hidden, int ffn, cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  BCHECK(checkShape(expertsLocal, cap, hidden, ffn, 1));
  if (!winSym || !a || !w) BFAIL(ncclInvalidArgument, "b200collEpGroupedGemm: null buffer");
  if (wRows <= 0 || wRows % 128 || K <= 0 || K % 8) BFAIL(ncclInvalidArgument, "b200collEpGroupedGemm: weight rows %% 128 and K %% 8 must be 0");
  if (!out && wRows != hidden) BFAIL(ncclInvalidArgument, "b200collEpGroupedGemm: the window's output region holds rows of `hidden` columns");
  EpGuard g(c->cudaDev);
  const EpLayout L = makeLayout(c->nranks, expertsLocal, cap, hidden, ffn);
  int parity;
  BCHECK(epLatestParity("b200collEpGroupedGemm", c, winSym, &parity));
  const uint32_t* cnt = (const uint32_t*)((const char*)winSym + L.cntOff) + (size_t)parity * expertsLocal;
  const int rows = expertsLocal * cap;
  const int bn = wRows % 256 == 0 ? 256 : 128;
  __nv_bfloat16* o = out ? (__nv_bfloat16*)out : (__nv_bfloat16*)((char*)winSym + L.outOff);
  gemm::Params p{};
  if (!gemm::makeTileMap(&p.mapA, a, rows, K, K, gemm::BM, 2) || !gemm::makeTileMap(&p.mapB, w, (uint64_t)expertsLocal * wRows, K, K, bn, 2))
    BFAIL(ncclInvalidArgument, "b200collEpGroupedGemm: misaligned operands");
  p.M = rows; p.N = wRows; p.K = K; p.tilesM = rows / gemm::BM; p.tilesN = wRows / bn; p.err = gemm::errWord();
  cudaError_t e;
  if (bn == 256) e = launchGrouped(p, GroupPolicy<256, false>{cnt, expertsLocal, nullptr, cap, cap / gemm::BM, wRows, o, wRows, wRows}, stream);
  else e = launchGrouped(p, GroupPolicy<128, false>{cnt, expertsLocal, nullptr, cap, cap / gemm::BM, wRows, o, wRows, wRows}, stream);
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "b200collEpGroupedGemm: launch failed: %s", cudaGetErrorString(e));
  return ncclSuccess;
}

// d gate[t, r] = <dy[t], output row of expert (t, r)> at the tokens' home rank; the forward pass's expert outputs must still be
// in the window (no grouped GEMM has written its output region since the combine).
ncclResult_t b200collEpGateGrad(ncclComm_t comm, void* winSym, const void* dy, const int* topIdx, const int* sentSlot, float* dGate, int T, int k,
                                int expertsLocal, int cap, int hidden, int ffn, cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  BCHECK(checkShape(expertsLocal, cap, hidden, ffn, k));
  if (!winSym || !dy || !topIdx || !sentSlot || !dGate) BFAIL(ncclInvalidArgument, "b200collEpGateGrad: null buffer");
  EpGuard g(c->cudaDev);
  GateGradArgs a{};
  a.L = makeLayout(c->nranks, expertsLocal, cap, hidden, ffn);
  if (!epPeers(c, winSym, a.L.total, a.win)) BFAIL(ncclInvalidUsage, "b200collEpGateGrad: the window must be symmetric memory");
  a.dy = (const __nv_bfloat16*)dy; a.topIdx = topIdx; a.sentSlot = sentSlot; a.dGate = dGate; a.T = T; a.k = k;
  if (T == 0) return ncclSuccess;
  const int ctas = std::max(1, std::min((T * k + 7) / 8, 8 * gemm::smCount()));
  epGateGrad<<<ctas, 256, 0, stream>>>(a);
  BCUDA(cudaGetLastError());
  return ncclSuccess;
}

// Gradient with respect to the expert output rows, gathered at the experts' rank: dOut[row] = gate * dy[token] for every row
// of the latest dispatch. dySym [T, hidden] bf16 and gateSym [T, k] fp32 are symmetric memory that every rank filled before
// this call on its stream; a barrier inside orders those writes (and every rank's epGateGrad) before the pulls.
ncclResult_t b200collEpGatherGrad(ncclComm_t comm, void* winSym, const void* dySym, const void* gateSym, void* dOut, int T, int k, int expertsLocal,
                                  int cap, int hidden, int ffn, cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  BCHECK(checkShape(expertsLocal, cap, hidden, ffn, k));
  if (!winSym || !dySym || !gateSym || !dOut) BFAIL(ncclInvalidArgument, "b200collEpGatherGrad: null buffer");
  EpGuard g(c->cudaDev);
  GatherGradArgs a{};
  a.L = makeLayout(c->nranks, expertsLocal, cap, hidden, ffn);
  char* dyPeer[kMaxRanks];
  char* gatePeer[kMaxRanks];
  if (!epPeers(c, dySym, (size_t)T * hidden * 2, dyPeer) || !epPeers(c, gateSym, (size_t)T * k * 4, gatePeer))
    BFAIL(ncclInvalidUsage, "b200collEpGatherGrad: dy and the gate weights must lie in symmetric memory");
  for (int r = 0; r < c->nranks; r++) { a.dyPeer[r] = dyPeer[r]; a.gatePeer[r] = gatePeer[r]; }
  BCHECK(epLatestParity("b200collEpGatherGrad", c, winSym, &a.parity));
  a.win = (const char*)winSym; a.k = k; a.T = T; a.dOut = (__nv_bfloat16*)dOut;
  if (c->nranks > 1) BCHECK(b200collBarrier(comm, stream));
  epGatherGrad<<<4 * gemm::smCount(), 256, 0, stream>>>(a);
  BCUDA(cudaGetLastError());
  return ncclSuccess;
}

// Rows per local expert after the latest dispatch (host copy; synchronises the stream) and the
// number of rows dropped so far because an expert's buffer was full.
ncclResult_t b200collEpCounts(ncclComm_t comm, void* winSym, int expertsLocal, int cap, int hidden, int ffn, unsigned int* countsHost, int* droppedHost,
                              cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  EpGuard g(c->cudaDev);
  const EpLayout L = makeLayout(c->nranks, expertsLocal, cap, hidden, ffn);
  EpState st;
  {
    std::lock_guard<std::mutex> lk(gEpMu);
    auto it = gEp.find(std::make_pair(c, (const void*)winSym));
    if (it == gEp.end() || it->second.calls == 0) BFAIL(ncclInvalidUsage, "b200collEpCounts: no dispatch has run on this window");
    st = it->second;
  }
  const int parity = (int)((st.calls - 1) & 1);
  BCUDA(cudaStreamSynchronize(stream));
  if (countsHost) BCUDA(cudaMemcpy(countsHost, (const char*)winSym + L.cntOff + (size_t)parity * expertsLocal * 4, (size_t)expertsLocal * 4, cudaMemcpyDeviceToHost));
  if (droppedHost) BCUDA(cudaMemcpy(droppedHost, st.ticket + 4, 4, cudaMemcpyDeviceToHost));
  return ncclSuccess;
}

}  // extern "C"
