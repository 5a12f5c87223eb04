// FSDP gradient path: reduce-scatter of a bf16 gradient bucket fused with the fp32 cast and the
// 1/N scale. Every rank stages its bucket once, then reduces its own 1/N slice straight out of
// its peers' staging buffers with fp32 accumulation (the sum is never rounded to bf16) and writes
// the scaled fp32 result into the gradient shard the optimizer reads. One kernel per bucket;
// protocol (staging halves, per-CTA barriers, bounded waits) is that of the collective kernels.
#include <algorithm>

#include "../coll/prims.cuh"
#include "../core/comm.h"
#include "../trace/tracer.h"
#include "b200coll/api_trace.h"
#include "b200coll/fused.h"

namespace b200 {

struct RsCastArgs {
  const __nv_bfloat16* send;  // n * count elements
  float* recv;                // count elements
  size_t count;
  float scale;
  int stageHalf;
  size_t chunkBytes;          // bytes of one rank's slice per chunk (equalised by the host); 0 = a whole staging share
};

// Host side of a staged call: equal chunks of one rank's staging share (the kernel lays data out by the chunk capacity
// alone, so a short last chunk would leave most lanes idle), this call's staging half, and the communicator's parity
// advanced by the number of chunks. Every rank computes the same from the same arguments.
inline RsCastArgs rsCastStagedArgs(Comm* c, const void* sendBf16, float* recvF32, size_t recvcount, float scale) {
  const size_t bytes = recvcount * 2;
  const size_t capMax = (c->dev.stageBytes / c->nranks) & ~(size_t)15;
  const size_t k = (bytes + capMax - 1) / capMax;
  size_t cap = (((bytes + k - 1) / k) + 15) & ~(size_t)15;
  if (cap > capMax) cap = capMax;
  RsCastArgs a{(const __nv_bfloat16*)sendBf16, recvF32, recvcount, scale, (int)(c->stageParity & 1), cap};
  c->stageParity += (uint32_t)((bytes + cap - 1) / cap);
  return a;
}

__device__ __forceinline__ void accum8(const uint4& v, float (&acc)[8], bool first) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] = first ? f.x : acc[2 * i] + f.x;
    acc[2 * i + 1] = first ? f.y : acc[2 * i + 1] + f.y;
  }
}

template <int MAXR, int UN>
__device__ __forceinline__ void reduceUnits(const DevComm& c, size_t stOff, float* out, size_t outElems, size_t u0, int nt, float scale, bool outAligned) {
  uint4 v[UN][MAXR];
#pragma unroll
  for (int j = 0; j < UN; j++)
#pragma unroll
    for (int p = 0; p < MAXR; p++)
      if (p < c.nranks) v[j][p] = ldStream16(c.ws[p] + stOff + ((u0 + (size_t)j * nt) << 4));
#pragma unroll
  for (int j = 0; j < UN; j++) {
    float acc[8];
#pragma unroll
    for (int p = 0; p < MAXR; p++)
      if (p < c.nranks) accum8(v[j][p], acc, p == 0);
    const size_t e0 = (u0 + (size_t)j * nt) * 8;
    if (outAligned && e0 + 8 <= outElems) {
      float4* o = reinterpret_cast<float4*>(out + e0);
      o[0] = make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
      o[1] = make_float4(acc[4] * scale, acc[5] * scale, acc[6] * scale, acc[7] * scale);
    } else {
#pragma unroll
      for (int k = 0; k < 8; k++)
        if (e0 + k < outElems) out[e0 + k] = acc[k] * scale;
    }
  }
}

__global__ void __launch_bounds__(kReduceThreads) kReduceScatterCast(const __grid_constant__ DevComm c, const __grid_constant__ RsCastArgs a) {
  stampBegin(c);
  const int n = c.nranks, rank = c.rank, B = gridDim.x, b = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
  uint32_t epoch = c.local->barEpoch[b];
  const size_t total = a.count * 2;  // bytes of one rank's slice
  const size_t fullCap = (c.stageBytes / n) & ~(size_t)15;
  const size_t cap = (a.chunkBytes && a.chunkBytes < fullCap) ? a.chunkBytes : fullCap;
  // A lane's range follows the chunk capacity, not how full a chunk is: what this lane stages into
  // a half can then never overlap what another lane of a peer (which this lane does not
  // synchronise with) still reads there from two chunks earlier.
  const size_t perLane = (((cap + 15) >> 4) + B - 1) / B;
  const char* send = (const char*)a.send;
  int half = a.stageHalf;
  for (size_t off = 0; off < total; off += cap, half ^= 1) {
    const size_t cb = total - off < cap ? total - off : cap;
    const size_t U = (cb + 15) >> 4;
    const size_t stageBase = c.stageOff + (size_t)half * c.stageBytes;
    size_t lo = (size_t)b * perLane, hi;
    if (lo > U) lo = U;
    hi = lo + perLane < U ? lo + perLane : U;
    const size_t bytes = lo < hi ? (((hi << 4) < cb ? (hi << 4) : cb) - (lo << 4)) : 0;
    for (int i = 0; i < n; i++) {
      const int s = (rank + i) % n;
      if (bytes) ctaCopy(c.ws[rank] + stageBase + (size_t)s * cap + (lo << 4), send + (size_t)s * total + off + (lo << 4), bytes);
    }
    ctaBarrier(c, epoch);
    const size_t stOff = stageBase + (size_t)rank * cap;
    float* out = a.recv + off / 2;
    const size_t outElems = cb / 2;
    const bool outAligned = (((uintptr_t)out) & 15) == 0;
    size_t u = lo + tid;
    if (n <= 2) {
      for (; u + (size_t)3 * nt < hi; u += (size_t)4 * nt) reduceUnits<2, 4>(c, stOff, out, outElems, u, nt, a.scale, outAligned);
      for (; u < hi; u += nt) reduceUnits<2, 1>(c, stOff, out, outElems, u, nt, a.scale, outAligned);
    } else if (n <= 4) {
      for (; u + (size_t)3 * nt < hi; u += (size_t)4 * nt) reduceUnits<4, 4>(c, stOff, out, outElems, u, nt, a.scale, outAligned);
      for (; u < hi; u += nt) reduceUnits<4, 1>(c, stOff, out, outElems, u, nt, a.scale, outAligned);
    } else {
      for (; u + (size_t)nt < hi; u += (size_t)2 * nt) reduceUnits<8, 2>(c, stOff, out, outElems, u, nt, a.scale, outAligned);
      for (; u < hi; u += nt) reduceUnits<8, 1>(c, stOff, out, outElems, u, nt, a.scale, outAligned);
    }
  }
  if (tid == 0) c.local->barEpoch[b] = epoch;
  stampEnd(c);
}

// Zero-copy variant for gradient buffers that live in symmetric memory (the same offset of a
// b200collSymAlloc window on every rank): nothing is staged, every rank reads its slice straight
// out of the peers' buffers. One barrier before (every rank has finished writing its gradients:
// each launches this kernel behind its own backward pass) and one after (a rank's buffer may be
// overwritten by its next backward pass only once no peer reads it any more).
struct RsCastDirectArgs {
  const char* sendPeer[kMaxRanks];  // every rank's gradient buffer as mapped here
  float* recv;
  size_t count;                     // elements of one rank's slice; count * 2 is a multiple of 16
  float scale;
};

template <int MAXR, int UN>
__device__ __forceinline__ void reduceUnitsDirect(const RsCastDirectArgs& a, int n, size_t sliceOff, size_t u0, int nt) {
  uint4 v[UN][MAXR];
#pragma unroll
  for (int j = 0; j < UN; j++)
#pragma unroll
    for (int p = 0; p < MAXR; p++)
      if (p < n) v[j][p] = ldStream16(a.sendPeer[p] + sliceOff + ((u0 + (size_t)j * nt) << 4));
#pragma unroll
  for (int j = 0; j < UN; j++) {
    float acc[8];
#pragma unroll
    for (int p = 0; p < MAXR; p++)
      if (p < n) accum8(v[j][p], acc, p == 0);
    float4* o = reinterpret_cast<float4*>(a.recv + (u0 + (size_t)j * nt) * 8);  // recv is 16-byte aligned, whole units only
    o[0] = make_float4(acc[0] * a.scale, acc[1] * a.scale, acc[2] * a.scale, acc[3] * a.scale);
    o[1] = make_float4(acc[4] * a.scale, acc[5] * a.scale, acc[6] * a.scale, acc[7] * a.scale);
  }
}

__global__ void __launch_bounds__(kReduceThreads) kReduceScatterCastDirect(const __grid_constant__ DevComm c, const __grid_constant__ RsCastDirectArgs a) {
  stampBegin(c);
  const int n = c.nranks, rank = c.rank, B = gridDim.x, b = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
  uint32_t epoch = c.local->barEpoch[b];
  const size_t total = a.count * 2;  // bytes of one rank's slice
  const size_t sliceOff = (size_t)rank * total;
  size_t lo, hi;
  splitUnits(total >> 4, B, b, lo, hi);
  ctaBarrier(c, epoch);
  size_t u = lo + tid;
  if (n <= 2) {
    for (; u + (size_t)3 * nt < hi; u += (size_t)4 * nt) reduceUnitsDirect<2, 4>(a, n, sliceOff, u, nt);
    for (; u < hi; u += nt) reduceUnitsDirect<2, 1>(a, n, sliceOff, u, nt);
  } else if (n <= 4) {
    for (; u + (size_t)nt < hi; u += (size_t)2 * nt) reduceUnitsDirect<4, 2>(a, n, sliceOff, u, nt);
    for (; u < hi; u += nt) reduceUnitsDirect<4, 1>(a, n, sliceOff, u, nt);
  } else {
    for (; u + (size_t)nt < hi; u += (size_t)2 * nt) reduceUnitsDirect<8, 2>(a, n, sliceOff, u, nt);
    for (; u < hi; u += nt) reduceUnitsDirect<8, 1>(a, n, sliceOff, u, nt);
  }
  ctaBarrier(c, epoch);
  if (tid == 0) c.local->barEpoch[b] = epoch;
  stampEnd(c);
}

// n == 1: nothing to exchange, only the cast and the scale.
__global__ void __launch_bounds__(256) kCastScaleSolo(const __nv_bfloat16* in, float* out, size_t n, float scale) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = __bfloat162float(in[i]) * scale;
}

}  // namespace b200

#ifndef B200_EMU_KERNELS_ONLY  // the emulation of several ranks on one GPU takes the kernels above and brings its own host side
using namespace b200;

extern "C" ncclResult_t b200collReduceScatterCast(ncclComm_t comm, const void* sendBf16, float* recvF32, size_t recvcount, float scale, cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (recvcount == 0) return ncclSuccess;
  if (!sendBf16 || !recvF32) BFAIL(ncclInvalidArgument, "b200collReduceScatterCast: null buffer");
  if (((uintptr_t)sendBf16 & 1) || ((uintptr_t)recvF32 & 3)) BFAIL(ncclInvalidArgument, "b200collReduceScatterCast: misaligned buffer");
  if (c->asyncError.load() != ncclSuccess) BFAIL((ncclResult_t)c->asyncError.load(), "communicator is in an error state: %s", c->lastErr.c_str());
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != c->cudaDev) cudaSetDevice(c->cudaDev);
  cudaError_t e;
  Tracer* tr = c->tracer;
  TraceStamp* stamp = tr ? tr->begin(B200COLL_API_ID_ncclReduceScatter, ncclBfloat16, recvcount, recvcount * 2 * c->nranks) : nullptr;
  if (c->nranks == 1) {
    size_t blocks = std::min<size_t>((recvcount + 255) / 256, 148 * 8);
    kCastScaleSolo<<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)sendBf16, recvF32, recvcount, scale);
    e = cudaGetLastError();
  } else {
    const size_t bytes = recvcount * 2;
    DevComm dc = c->dev;
    size_t moved = recvcount * 2 * c->nranks;
    int ctas = (int)std::min<size_t>((moved + (64u << 10) - 1) / (64u << 10), (size_t)c->maxCtas);
    ctas = std::min(std::max(ctas, c->minCtas) * 2, kMaxCtas);
    // Gradient buffer inside a symmetric window, whole 16-byte units, aligned ends: read the peers in place.
    size_t woff = 0;
    Window* win = nullptr;
    if ((bytes & 15) == 0 && (((uintptr_t)sendBf16 | (uintptr_t)recvF32) & 15) == 0) {
      std::lock_guard<std::mutex> lk(c->mu);
      win = c->findWindow(sendBf16, bytes * c->nranks, &woff);
    }
    if (win) {
      RsCastDirectArgs da{};
      for (int p = 0; p < c->nranks; p++) da.sendPeer[p] = win->seg.peer[p] + woff;
      da.recv = recvF32;
      da.count = recvcount;
      da.scale = scale;
      dc.opSeq = ++c->opSeq;
      dc.stamp = stamp;
      if (tr) tr->setAlgo(ALGO_P2P, ctas);
      kReduceScatterCastDirect<<<ctas, kReduceThreads, 0, stream>>>(dc, da);
      e = cudaGetLastError();
      if (tr) tr->end(e == cudaSuccess);
      if (prev != c->cudaDev && prev >= 0) cudaSetDevice(prev);
      if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "b200collReduceScatterCast launch failed: %s", cudaGetErrorString(e));
      return ncclSuccess;
    }
    const RsCastArgs a = rsCastStagedArgs(c, sendBf16, recvF32, recvcount, scale);
    dc.opSeq = ++c->opSeq;
    dc.stamp = stamp;
    if (tr) tr->setAlgo(ALGO_P2P, ctas);
    kReduceScatterCast<<<ctas, kReduceThreads, 0, stream>>>(dc, a);
    e = cudaGetLastError();
  }
  if (tr) tr->end(e == cudaSuccess);
  if (prev != c->cudaDev && prev >= 0) cudaSetDevice(prev);
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "b200collReduceScatterCast launch failed: %s", cudaGetErrorString(e));
  return ncclSuccess;
}
#endif  // B200_EMU_KERNELS_ONLY
