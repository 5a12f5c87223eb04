// The collective kernels (sm_100a). One launch per collective call; CTA `b` of every rank forms
// an independent lane that synchronises only with CTA `b` of its peers.
//
// Algorithms, by message size (semantics: rccl.h:548-934; in-place rules rccl.h:665-705):
//   kLLAllReduce      one-shot all-reduce for small messages: every rank stores its data into
//                     every peer's buffer as 16-byte lines {data, flag, data, flag}; the flag in
//                     the line is the only synchronisation (one NVLink crossing of latency).
//   kStagedReduce     AllReduce / ReduceScatter / Reduce through a symmetric staging buffer,
//                     software-pipelined over chunks: while half of the CTA reduces chunk k over
//                     NVLink (one multimem.ld_reduce that adds inside the NVSwitch, or bulk
//                     asynchronous copies of every rank's tile into a shared-memory ring), the
//                     other half copies chunk k-1 out of staging and chunk k+1 into it. Results go
//                     straight to where they are needed (multimem.st / peer stores / local recv).
//                     With registered symmetric buffers the copies disappear.
//   kStagedCopy       AllGather (pull from peers' staging into recv, pipelined the same way
//                     between few ranks; short parts are pulled from all peers at once) and
//                     Broadcast (root fills staging, with one multicast store when NVLS is on;
//                     the others copy out).
//   kP2p              grouped Send/Recv work list over per-peer FIFOs with credits; AllToAll(v),
//                     Gather and Scatter are built from it.
// Staging halves alternate per chunk; every chunk's copy-in is followed by a full barrier before
// anyone reads it, which is what makes reusing a half two chunks later safe without a trailing
// barrier, also across calls. Where data of a chunk lives in a half, and which lane handles it,
// depends on the chunk capacity alone (see the note on geometry in kStagedReduce).
#pragma once

#include <type_traits>

#include "prims.cuh"
#include "reduce_ops.cuh"

namespace b200 {

// ---- element-wise helpers (tails and unaligned buffers) -------------------------------------
template <typename T>
__device__ __forceinline__ void loadUnit8(const T* base, size_t count, size_t unit, bool aligned, T (&e)[8 / sizeof(T)]) {
  constexpr int EPU = 8 / sizeof(T);
  const size_t i0 = unit * EPU;
  if (aligned && i0 + EPU <= count) {
    union { uint2 v; T t[EPU]; } u;
    u.v = *(const uint2*)(base + i0);
#pragma unroll
    for (int k = 0; k < EPU; k++) e[k] = u.t[k];
  } else {
#pragma unroll
    for (int k = 0; k < EPU; k++) {
      if (i0 + k < count) e[k] = base[i0 + k];
      else e[k] = ElemTraits<T>::down(typename ElemTraits<T>::Acc(0));
    }
  }
}

// PreMulSum multiplies a rank's own input by that rank's scalar, so the scaling happens where
// the input is read (before it is sent or staged), never on the reducing side.
template <typename T>
__device__ __forceinline__ T preMul(T v, typename ElemTraits<T>::Acc scalar) {
  return ElemTraits<T>::down(ElemTraits<T>::up(v) * scalar);
}

template <typename T, typename Op>
__global__ void __launch_bounds__(kCollThreads) kLLAllReduce(const __grid_constant__ DevComm c, const __grid_constant__ LLArgs a) {
  stampBegin(c);
  constexpr int EPU = 8 / sizeof(T);
  using Acc = typename ElemTraits<T>::Acc;
  const int n = c.nranks, rank = c.rank;
  const size_t units = (a.count + EPU - 1) / EPU;
  const size_t halfOff = kWsLLOff + (size_t)(a.seq & 1) * (size_t)n * c.llSlotBytes;
  // Reduce-scatter is the same exchange with one slice per destination: rank p gets slice p of everybody's input and
  // nobody else's, so every line crosses the link once.
  const bool rs = a.kind == COLL_REDUCESCATTER;
  const T* send = (const T*)a.send;
  T* recv = (T*)a.recv;
  const bool aligned = ((((uintptr_t)a.send) | ((uintptr_t)a.recv)) & 7) == 0 && (!rs || (a.count * sizeof(T)) % 8 == 0);
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t gn = (size_t)gridDim.x * blockDim.x;

  const Acc scalar = scalarOf<T>(a.scalarBits, a.scalarPtr);
  const bool pre = a.scaleMode == SCALE_PRE_MUL;
  if (rs) {
    for (size_t i = gtid; i < units; i += gn) {
      for (int d = 1; d < n; d++) {
        const int p = (rank + d) % n;
        T e[EPU];
        loadUnit8<T>(send + (size_t)p * a.count, a.count, i, aligned, e);
        union { uint2 v; T t[EPU]; } u;
#pragma unroll
        for (int k = 0; k < EPU; k++) u.t[k] = pre ? preMul<T>(e[k], scalar) : e[k];
        stVolatile16(c.ws[p] + halfOff + (size_t)rank * c.llSlotBytes + i * 16, make_uint4(u.v.x, a.seq, u.v.y, a.seq));
      }
    }
    send += (size_t)rank * a.count;  // this rank's own contribution to its slice
  } else {
    for (size_t i = gtid; i < units; i += gn) {
      T e[EPU];
      loadUnit8<T>(send, a.count, i, aligned, e);
      union { uint2 v; T t[EPU]; } u;
#pragma unroll
      for (int k = 0; k < EPU; k++) u.t[k] = pre ? preMul<T>(e[k], scalar) : e[k];
      const uint4 line = make_uint4(u.v.x, a.seq, u.v.y, a.seq);
      for (int d = 1; d < n; d++) {
        const int p = (rank + d) % n;
        stVolatile16(c.ws[p] + halfOff + (size_t)rank * c.llSlotBytes + i * 16, line);
      }
    }
  }

  for (size_t i = gtid; i < units; i += gn) {
    Acc acc[EPU];
    for (int s = 0; s < n; s++) {
      union { uint2 v; T t[EPU]; } u;
      if (s == rank) {
        T e[EPU];
        loadUnit8<T>(send, a.count, i, aligned, e);
#pragma unroll
        for (int k = 0; k < EPU; k++) u.t[k] = pre ? preMul<T>(e[k], scalar) : e[k];
      } else {
        const char* line = c.ws[rank] + halfOff + (size_t)s * c.llSlotBytes + i * 16;
        uint4 v;
        unsigned long long t0 = 0;
        uint32_t spins = 0;
        bool ok = true;
        while (true) {
          v = ldVolatile16(line);
          if (v.y == a.seq && v.w == a.seq) break;
          if ((++spins & 0xff) == 0) {
            if (*(volatile uint32_t*)&c.local->failed) { ok = false; break; }
            if (*c.abortFlag) { recordFailure(c, 2, WAIT_LL, s, a.seq, v.y); ok = false; break; }
            unsigned long long now = globalTimerNs();
            if (t0 == 0) t0 = now;
            else if (now - t0 > c.timeoutNs) { recordFailure(c, 1, WAIT_LL, s, a.seq, v.y); ok = false; break; }
          }
        }
        u.v = ok ? make_uint2(v.x, v.z) : make_uint2(0, 0);
      }
#pragma unroll
      for (int k = 0; k < EPU; k++) {
        Acc x = ElemTraits<T>::up(u.t[k]);
        acc[k] = (s == 0) ? x : Op::apply(acc[k], x);
      }
    }
    const size_t i0 = i * EPU;
    union { uint2 v; T t[EPU]; } o;
#pragma unroll
    for (int k = 0; k < EPU; k++) {
      Acc x = acc[k];
      if (a.scaleMode == SCALE_POST_DIV_N) x = postDiv<T>(x, n);
      o.t[k] = ElemTraits<T>::down(x);
    }
    if (aligned && i0 + EPU <= a.count) {
      *(uint2*)(recv + i0) = o.v;
    } else {
#pragma unroll
      for (int k = 0; k < EPU; k++)
        if (i0 + k < a.count) recv[i0 + k] = o.t[k];
    }
  }
  stampEnd(c);
}

// ---- staged / direct reduce -----------------------------------------------------------------
// Store 16 bytes of results to a local user buffer that may be unaligned or end mid-unit.
template <typename T>
__device__ __forceinline__ void storeUser16(char* base, size_t byteOff, size_t limitBytes, uint4 v, bool aligned) {
  if (aligned && byteOff + 16 <= limitBytes) {
    st16(base + byteOff, v);
  } else {
    union { uint4 v; T t[16 / sizeof(T)]; } u;
    u.v = v;
#pragma unroll
    for (int k = 0; k < (int)(16 / sizeof(T)); k++)
      if (byteOff + (k + 1) * sizeof(T) <= limitBytes) *(T*)(base + byteOff + k * sizeof(T)) = u.t[k];
  }
}

// Copy into staging while multiplying by this rank's PreMulSum scalar (staging is 16-byte
// aligned; the user buffer may not be).
template <typename T>
__device__ __forceinline__ void ctaCopyScaled(char* dst, const char* src, size_t bytes, typename ElemTraits<T>::Acc scalar, const int t, const int nt) {
  using P = Pack<T>;
  if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
    const size_t nvec = bytes >> 4;
    for (size_t i = t; i < nvec; i += nt) {
      typename P::Acc a[P::N];
      P::up(ldStream16(src + (i << 4)), a);
#pragma unroll
      for (int k = 0; k < P::N; k++) a[k] = a[k] * scalar;
      st16(dst + (i << 4), P::down(a));
    }
    for (size_t b = (nvec << 4) + (size_t)t * sizeof(T); b + sizeof(T) <= bytes; b += (size_t)nt * sizeof(T))
      *(T*)(dst + b) = preMul<T>(*(const T*)(src + b), scalar);
  } else {
    for (size_t b = (size_t)t * sizeof(T); b + sizeof(T) <= bytes; b += (size_t)nt * sizeof(T))
      *(T*)(dst + b) = preMul<T>(*(const T*)(src + b), scalar);
  }
}

// Staged mode is software-pipelined over chunks: while one half of the CTA's threads reduces chunk
// k over NVLink, the other half copies chunk k-1's results out of staging and chunk k+1's input
// into it (both local HBM traffic), with one inter-rank barrier per chunk:
//
//     copyIn(0) | barrier | { reduce(k)  ||  copyOut(k-1); copyIn(k+1) } barrier | ... | copyOut(last)
//
// Chunk k lives in staging half (first + k) & 1. reduce(k) touches every rank's half k; the copies
// touch only this rank's other half, which nobody reads remotely between the barriers around them.
template <typename T, typename Op, bool NVLS>
__global__ void __launch_bounds__(NVLS ? kCollThreads : kReduceThreads) kStagedReduce(const __grid_constant__ DevComm c, const __grid_constant__ CollArgs a) {
  stampBegin(c);
  using P = Pack<T>;
  using Acc = typename ElemTraits<T>::Acc;
  constexpr size_t ES = sizeof(T);
  const int n = c.nranks, rank = c.rank, B = gridDim.x, b = blockIdx.x;
  const int tid = threadIdx.x, nt = blockDim.x;
  uint32_t epoch = c.local->barEpoch[b];
  const bool isRS = a.kind == COLL_REDUCESCATTER;
  const bool isAR = a.kind == COLL_ALLREDUCE;
  const bool isRed = a.kind == COLL_REDUCE;
  const size_t total = a.count * ES;  // AllReduce/Reduce: the message; ReduceScatter: one rank's slice
  const size_t fullCap = isRS ? (c.stageBytes / n) & ~(size_t)15 : c.stageBytes;
  const size_t cap = a.direct ? ((total + 15) & ~(size_t)15) : ((a.chunkBytes && a.chunkBytes < fullCap) ? a.chunkBytes : fullCap);
  const Acc scalar = scalarOf<T>(a.scalarBits, a.scalarPtr);
  const char* send = (const char*)a.send;
  char* recv = (char*)a.recv;
  // The slice this rank reduces never needs to pass through its own staging: its copy is read straight from the user's
  // send buffer (and, in an all-reduce, the result stored straight into the user's receive buffer). That takes 1/n of the
  // copy-in and of the copy-out away: between two ranks the local copies, not NVLink, bound the large messages. Needs
  // whole 16-byte units (the bulk loads read whole units) and no scaling while staging.
  const bool ownDirect = !NVLS && !a.direct && a.scaleMode != SCALE_PRE_MUL && (((uintptr_t)send) & 15) == 0 && (total & 15) == 0;

  // Shared-memory ring of the peer-load path (kernels without in-switch reduction only).
  extern __shared__ __align__(128) unsigned char bulkSmem[];
  uint64_t* bulkFull = reinterpret_cast<uint64_t*>(bulkSmem);
  char* bulkStage = reinterpret_cast<char*>(bulkSmem) + 128;
  uint32_t tileSeq = 0;     // tiles consumed so far by this CTA (same value in every thread)
  uint32_t bulkIssued = 0;  // tiles issued so far (meaningful in the issuing thread)
  if constexpr (!NVLS) {
    if (tid == 0) {
      for (int i = 0; i < kBulkStages; i++) cmbarInit(&bulkFull[i], 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
  }

  // Geometry of the chunk that starts at byte `off` (per slice for ReduceScatter).
  // Geometry. Where a piece of a chunk lives in staging, and which lane (CTA index) handles it,
  // depends only on the chunk capacity `cap`, never on how full a chunk is: a lane's ranges of a
  // short last chunk then lie inside its ranges of a full one, so what one lane writes into a
  // staging half can never overlap what another lane (which it does not synchronise with) still
  // reads there from an earlier chunk.
  struct Geo {
    size_t off, cb, stageBase;
  };
  const size_t capUnits = (cap + 15) >> 4;
  const size_t su = isRS ? capUnits : (capUnits + n - 1) / n;  // 16-byte units per slice of a full chunk
  const size_t perLane = (su + B - 1) / B;                      // units of a slice per lane
  auto geo = [&](size_t off, int half) -> Geo {
    Geo g;
    g.off = off;
    g.cb = (total - off < cap) ? total - off : cap;
    g.stageBase = c.stageOff + (size_t)half * c.stageBytes;
    return g;
  };
  auto sliceBytes = [&](const Geo& g, int s) -> size_t {
    if (isRS) return g.cb;
    size_t lo = (size_t)s * su * 16;
    if (lo >= g.cb) return 0;
    size_t len = g.cb - lo;
    return len < su * 16 ? len : su * 16;
  };
  // This lane's units [lo, hi) of a slice that holds `sb` bytes.
  auto laneRange = [&](size_t sb, size_t& lo, size_t& hi) {
    const size_t units = (sb + 15) >> 4;
    lo = (size_t)b * perLane;
    if (lo > units) lo = units;
    hi = lo + perLane;
    if (hi > units) hi = units;
  };
  auto sliceStage = [&](const Geo&, int s) -> size_t { return isRS ? (size_t)s * cap : (size_t)s * su * 16; };
  auto sliceSrc = [&](const Geo& g, int s) -> const char* {
    return isRS ? send + ((size_t)s * a.count * ES + g.off) : send + g.off + (size_t)s * su * 16;
  };

  // user send -> this rank's staging, by threads t of nt
  auto copyIn = [&](const Geo& g, int t, int ntg) {
    for (int i = ownDirect ? 1 : 0; i < n; i++) {
      const int s = (rank + i) % n;
      const size_t sb = sliceBytes(g, s);
      size_t lo, hi;
      laneRange(sb, lo, hi);
      if (lo < hi) {
        size_t bytes = ((hi << 4) < sb ? (hi << 4) : sb) - (lo << 4);
        char* dst = c.ws[rank] + g.stageBase + sliceStage(g, s) + (lo << 4);
        if (a.scaleMode == SCALE_PRE_MUL) ctaCopyScaled<T>(dst, sliceSrc(g, s) + (lo << 4), bytes, scalar, t, ntg);
        else groupCopy(dst, sliceSrc(g, s) + (lo << 4), bytes, t, ntg);
      }
    }
  };
  // this rank's staging -> user recv (AllReduce; Reduce root without NVLS)
  auto copyOut = [&](const Geo& g, int t, int ntg) {
    for (int i = (ownDirect && isAR) ? 1 : 0; i < n; i++) {
      const int s = (rank + i) % n;
      const size_t sb = sliceBytes(g, s);
      size_t lo, hi;
      laneRange(sb, lo, hi);
      if (lo < hi) {
        size_t bytes = ((hi << 4) < sb ? (hi << 4) : sb) - (lo << 4);
        groupCopy(recv + g.off + (size_t)s * su * 16 + (lo << 4), c.ws[rank] + g.stageBase + sliceStage(g, s) + (lo << 4), bytes, t, ntg);
      }
    }
  };

  // Reduce. Normally this rank reduces slice `rank`; the NVLS Reduce root pulls every slice.
  auto reduceChunk = [&](const Geo& g, const int t, const int ntg) {
    const size_t off = g.off;
    const bool pullAll = NVLS && isRed;
    if (pullAll && rank != a.root) return;
    for (int si = 0; si < (pullAll ? n : 1); si++) {
      const int s = pullAll ? si : rank;
      const size_t sb = sliceBytes(g, s);
      size_t lo, hi;
      laneRange(sb, lo, hi);
      // Byte offset of the slice inside the message (direct windows and user recv).
      const size_t msgOff = isRS ? off : off + (size_t)s * su * 16;
      const size_t stOff = g.stageBase + sliceStage(g, s);
      const bool recvAligned = (((uintptr_t)(recv + (isRS ? off : msgOff))) & 15) == 0;
      // Sources and destinations of this slice.
      const size_t srcOff = isRS ? (size_t)s * a.count * ES + off : msgOff;
      const char* mcSrc = NVLS ? (a.direct ? a.sendMc + srcOff : c.wsMc + stOff) : nullptr;
      char* mcDst = (NVLS && isAR) ? (a.direct ? a.recvMc + msgOff : c.wsMc + stOff) : nullptr;
      // Peer bases come from the kernel parameters (constant bank), indexed by unrolled loops.
      auto pSrc = [&](int p) -> const char* {
        if (a.direct) return a.sendPeer[p] + srcOff;
        return (ownDirect && p == rank) ? send + srcOff : c.ws[p] + stOff;
      };
      auto pDst = [&](int p) -> char* { return a.direct ? a.recvPeer[p] + msgOff : c.ws[p] + stOff; };
      auto deliver = [&](size_t u, uint4 out) {
        if (isRS) {
          storeUser16<T>(recv, off + (u << 4), total, out, recvAligned);
        } else if (isAR) {
          if constexpr (NVLS) {
            mcStore16(mcDst + (u << 4), out);
          } else {
#pragma unroll
            for (int p = 0; p < kMaxRanks; p++)
              if (p < n && !(ownDirect && p == rank)) st16(pDst(p) + (u << 4), out);
            if (ownDirect) storeUser16<T>(recv, msgOff + (u << 4), total, out, recvAligned);
          }
        } else {  // Reduce
          if constexpr (NVLS) storeUser16<T>(recv, msgOff + (u << 4), total, out, recvAligned);
          else st16(pDst(a.root) + (u << 4), out);
        }
      };
      if constexpr (NVLS) {
        // One switch-side reduction per 16-byte unit; eight are in flight per thread.
        auto body = [&](auto unTag, size_t u0) {
          constexpr int UN = decltype(unTag)::value;
          uint4 out[UN];
#pragma unroll
          for (int j = 0; j < UN; j++) out[j] = McReduce<T>::ld(mcSrc + ((u0 + (size_t)j * ntg) << 4));
          if (a.scaleMode == SCALE_POST_DIV_N) {
#pragma unroll
            for (int j = 0; j < UN; j++) {
              Acc acc[P::N];
              P::up(out[j], acc);
#pragma unroll
              for (int k = 0; k < P::N; k++) acc[k] = postDiv<T>(acc[k], n);
              out[j] = P::down(acc);
            }
          }
#pragma unroll
          for (int j = 0; j < UN; j++) deliver(u0 + (size_t)j * ntg, out[j]);
        };
        size_t u = lo + t;
        for (; u + (size_t)7 * ntg < hi; u += (size_t)8 * ntg) body(std::integral_constant<int, 8>{}, u);
        for (; u < hi; u += ntg) body(std::integral_constant<int, 1>{}, u);
      } else {
        // Peer loads as bulk asynchronous copies: thread 0 of the group keeps kBulkStages - 1
        // tiles (every rank's copy of the same range) in flight into a shared-memory ring; all
        // threads reduce a landed tile from shared memory and send the result on its way.
        const uint32_t tileBytes = kBulkStageBytes / (n <= 2 ? 2 : (n <= 4 ? 4 : 8));
        const size_t rangeBytes = (hi - lo) << 4;
        const uint32_t tiles = (uint32_t)((rangeBytes + tileBytes - 1) / tileBytes);
        auto issue = [&](uint32_t i) {
          const uint32_t seq = tileSeq + i, st = seq % kBulkStages;
          const size_t left = rangeBytes - (size_t)i * tileBytes;
          const uint32_t tb = left < tileBytes ? (uint32_t)left : tileBytes;
          // The stage was last read, and the sources last written (by copy-in here or on a peer,
          // ordered before this point by the inter-rank barrier), through the generic proxy.
          asm volatile("fence.proxy.async;" ::: "memory");
          cmbarExpectTx(&bulkFull[st], tb * (uint32_t)n);
          for (int p = 0; p < n; p++)
            bulkLoad(bulkStage + (size_t)st * kBulkStageBytes + (size_t)p * tileBytes, pSrc(p) + (lo << 4) + (size_t)i * tileBytes, tb, &bulkFull[st]);
          bulkIssued = seq + 1;
        };
        if (t == 0)
          for (uint32_t i = 0; i < tiles && i < (uint32_t)kBulkStages - 1; i++) issue(i);
        for (uint32_t i = 0; i < tiles; i++) {
          const uint32_t seq = tileSeq + i, st = seq % kBulkStages;
          const bool ok = cmbarWaitBounded(c, &bulkFull[st], (seq / kBulkStages) & 1, (uint32_t)rank);
          // The stage read in the previous iteration is free: everyone passed the barrier below.
          if (t == 0 && ok && i + kBulkStages - 1 < tiles) issue(i + kBulkStages - 1);
          if (ok) {
            const size_t left = rangeBytes - (size_t)i * tileBytes;
            const uint32_t units = (uint32_t)((left < tileBytes ? left : tileBytes) >> 4);
            const char* stage = bulkStage + (size_t)st * kBulkStageBytes;
            const size_t ubase = lo + (size_t)i * (tileBytes >> 4);
            for (uint32_t uu = t; uu < units; uu += ntg) {
              Acc acc[P::N];
#pragma unroll
              for (int p = 0; p < kMaxRanks; p++) {
                if (p < n) {
                  Acc x[P::N];
                  P::up(*reinterpret_cast<const uint4*>(stage + (size_t)p * tileBytes + ((size_t)uu << 4)), x);
#pragma unroll
                  for (int k = 0; k < P::N; k++) acc[k] = (p == 0) ? x[k] : Op::apply(acc[k], x[k]);
                }
              }
              if (a.scaleMode == SCALE_POST_DIV_N) {
#pragma unroll
                for (int k = 0; k < P::N; k++) acc[k] = postDiv<T>(acc[k], n);
              }
              deliver(ubase + uu, P::down(acc));
            }
          }
          asm volatile("bar.sync 2, %0;" ::"r"(ntg) : "memory");
        }
      }
    }
  };

  // Zero-copy windows (direct) are one chunk with no copies: a barrier before (inputs complete
  // everywhere) and after (nobody leaves while a peer still reads its buffer or has stores to it
  // in flight).
  // Tiles the peer-load path consumes for this CTA's share of slice `rank` of a chunk.
  auto tilesOf = [&](const Geo& g) -> uint32_t {
    const size_t sb = sliceBytes(g, rank);
    size_t lo, hi;
    laneRange(sb, lo, hi);
    const uint32_t tileBytes = kBulkStageBytes / (n <= 2 ? 2 : (n <= 4 ? 4 : 8));
    return (uint32_t)((((hi - lo) << 4) + tileBytes - 1) / tileBytes);
  };
  const bool hasOut = !a.direct && (isAR || (isRed && !NVLS && rank == a.root));  // results come back through staging
  const bool barAfter = a.direct || isAR || (isRed && !NVLS);                     // every chunk's reduce ends with a barrier
  int half = a.direct ? 0 : a.stageHalf;
  if (!a.direct) copyIn(geo(0, half), tid, nt);
  ctaBarrier(c, epoch);
  for (size_t off = 0; off < total; off += cap, half ^= 1) {
    const Geo g = geo(off, half);
    const bool more = off + cap < total;
    const bool prevOut = hasOut && off > 0;
    // With local copies to overlap, the lower half of the CTA reduces over NVLink and the upper
    // half copies; otherwise every thread reduces.
    // (three quarters reduce when the rank's own slice bypasses staging: the copies have 1/n less to move, and between
    // two ranks the reducing threads, not the copies, were the slower group)
    const int h = (more || prevOut) ? (ownDirect ? (nt * 3) >> 2 : nt >> 1) : nt;
    if (tid < h) {
      reduceChunk(g, tid, h);
    } else {
      if (prevOut) {
        copyOut(geo(off - cap, half ^ 1), tid - h, nt - h);
        // the copy-in below overwrites what other threads of this group have just read
        asm volatile("bar.sync 1, %0;" ::"r"(nt - h) : "memory");
      }
      if (more) copyIn(geo(off + cap, half ^ 1), tid - h, nt - h);
    }
    if constexpr (!NVLS) tileSeq += tilesOf(g);
    if (barAfter || more) ctaBarrier(c, epoch);
    if (!more && hasOut) copyOut(g, tid, nt);
  }
  if constexpr (!NVLS) {
    // After a wait that was given up, copies may still be on their way into this CTA's shared
    // memory: give each issued tile one more bounded wait before the CTA ends.
    if (tid == 0 && *(volatile uint32_t*)&c.local->failed) {
      for (uint32_t seq = bulkIssued > (uint32_t)kBulkStages ? bulkIssued - kBulkStages : 0; seq < bulkIssued; seq++)
        for (uint32_t spin = 0; spin < (1u << 16) && !cmbarTryWait(&bulkFull[seq % kBulkStages], (seq / kBulkStages) & 1); spin++) {
        }
    }
  }
  if (tid == 0) c.local->barEpoch[b] = epoch;
  stampEnd(c);
}

// ---- staged / direct copy collectives: AllGather and Broadcast ------------------------------
__device__ __forceinline__ void ctaCopyToMc(char* mcDst, const char* src, size_t bytes) {
  // Multicast store of whole 16-byte units (staging is padded, so rounding up is safe).
  const size_t nvec = (bytes + 15) >> 4;
  const bool aligned = (((uintptr_t)src) & 15) == 0;
  size_t i = threadIdx.x;
  if (aligned) {
    // whole units with eight loads in flight per thread; the ragged end goes through the loop below
    const size_t whole = bytes >> 4;
    constexpr int U = 8;
    const size_t nt = blockDim.x;
    for (; i + (U - 1) * nt < whole; i += U * nt) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; u++) v[u] = ldStream16(src + ((i + u * nt) << 4));
#pragma unroll
      for (int u = 0; u < U; u++) mcStore16(mcDst + ((i + u * nt) << 4), v[u]);
    }
  }
  for (; i < nvec; i += blockDim.x) {
    uint4 v;
    if (aligned && ((i + 1) << 4) <= bytes) {
      v = ldStream16(src + (i << 4));
    } else {
      union { uint4 v; unsigned char c[16]; } u;
      u.v = make_uint4(0, 0, 0, 0);
      for (int k = 0; k < 16; k++)
        if ((i << 4) + k < bytes) u.c[k] = ((const unsigned char*)src)[(i << 4) + k];
      v = u.v;
    }
    mcStore16(mcDst + (i << 4), v);
  }
}

template <bool NVLS>
__global__ void __launch_bounds__(kCollThreads) kStagedCopy(const __grid_constant__ DevComm c, const __grid_constant__ CollArgs a, const int elemSize) {
  stampBegin(c);
  const int n = c.nranks, rank = c.rank, B = gridDim.x, b = blockIdx.x;
  uint32_t epoch = c.local->barEpoch[b];
  const size_t total = a.count * (size_t)elemSize;  // AllGather: one rank's contribution; Broadcast: the message
  const bool isA2A = a.kind == COLL_ALLTOALL;
  // All-to-all: a staging half holds one slot per source rank; a step moves at most a slot of every pair's chunk.
  const size_t slotCap = (c.stageBytes / (size_t)n) & ~(size_t)15;
  const size_t cap = isA2A ? (((total + 15) & ~(size_t)15) < slotCap ? ((total + 15) & ~(size_t)15) : slotCap)
                           : (a.direct ? ((total + 15) & ~(size_t)15) : ((a.chunkBytes && a.chunkBytes < c.stageBytes) ? a.chunkBytes : c.stageBytes));
  const char* send = (const char*)a.send;
  char* recv = (char*)a.recv;
  int half = a.stageHalf;
  const bool isAG = a.kind == COLL_ALLGATHER;

  // This CTA's part of the chunk at `off`: byte offset inside the chunk and length.
  // The lane's range is fixed by the chunk capacity, not by how full the chunk is (see the note
  // on geometry in kStagedReduce): lanes never touch one another's part of a staging half.
  const size_t perLane = (((cap + 15) >> 4) + B - 1) / B;
  auto part = [&](size_t off, size_t& bo, size_t& bytes) {
    const size_t cb = (total - off < cap) ? total - off : cap;
    const size_t units = (cb + 15) >> 4;
    size_t lo = (size_t)b * perLane, hi;
    if (lo > units) lo = units;
    hi = lo + perLane < units ? lo + perLane : units;
    bytes = lo < hi ? (((hi << 4) < cb ? (hi << 4) : cb) - (lo << 4)) : 0;
    bo = lo << 4;
  };
  if (isAG && !a.direct) {
    // Staged all-gather, pipelined like the staged reduce: while the lower half of the CTA pulls
    // chunk k from the peers' staging over NVLink, the upper half copies this rank's own part
    // to its place in recv and stages chunk k+1 (both local). One barrier per chunk.
    const int tid = threadIdx.x, nt = blockDim.x;
    size_t bo, bytes;
    part(0, bo, bytes);
    ctaCopy(c.ws[rank] + c.stageOff + (size_t)half * c.stageBytes + bo, send + bo, bytes);
    ctaBarrier(c, epoch);
    for (size_t off = 0; off < total; off += cap, half ^= 1) {
      const size_t stageBase = c.stageOff + (size_t)half * c.stageBytes;
      part(off, bo, bytes);
      const bool more = off + cap < total;
      const bool selfCopy = recv + (size_t)rank * total != send;
      // The local copies are 2/(n-1) of the bytes the pulls move: worth half the CTA's threads
      // only between few ranks, and only when there is a next chunk to stage meanwhile.
      const bool split = more && n <= 4;
      const int h = split ? nt >> 1 : nt;
      const int warps = h >> 5, peers = n - 1;
      if (tid < h) {
        if (bytes <= (size_t)(64u << 10) && warps >= peers && peers > 1) {
          // Short parts: pulling peer after peer would pay one NVLink round trip per peer in
          // sequence, so the warps share out the peers and all pulls are in flight together.
          const int per = warps / peers;              // warps per peer
          const int w = tid >> 5;
          if (w < per * peers) {
            const int p = (rank + 1 + w / per) % n;
            groupCopy(recv + (size_t)p * total + off + bo, c.ws[p] + stageBase + bo, bytes, (w % per) * 32 + (tid & 31), per * 32);
          }
        } else {
          for (int i = 1; i < n; i++) {
            const int p = (rank + i) % n;
            groupCopy(recv + (size_t)p * total + off + bo, c.ws[p] + stageBase + bo, bytes, tid, h);
          }
        }
      }
      if (tid >= h || !split) {
        const int t2 = split ? tid - h : tid, n2 = split ? nt - h : nt;
        if (selfCopy) groupCopy(recv + (size_t)rank * total + off + bo, send + off + bo, bytes, t2, n2);
        if (more) {
          size_t nbo, nbytes;
          part(off + cap, nbo, nbytes);
          groupCopy(c.ws[rank] + c.stageOff + (size_t)(half ^ 1) * c.stageBytes + nbo, send + off + cap + nbo, nbytes, t2, n2);
        }
      }
      if (more) ctaBarrier(c, epoch);
    }
    if (threadIdx.x == 0) c.local->barEpoch[b] = epoch;
    stampEnd(c);
    return;
  }

  if (isA2A) {
    // Staged all-to-all for large chunks (total = bytes per pair): every rank stores its piece for peer p into slot
    // `rank` of p's staging half (plain peer stores, the fast direction of the link); after a barrier everybody copies
    // its slots out of its OWN half. Software pipeline: three quarters of a CTA's threads push step k+1 into the other
    // half while the last quarter copies step k out (and, in the first step, makes the rank's own block), one barrier per
    // step. A half is written again two steps later, behind a barrier that every rank reaches after its copy-out.
    const int nt = blockDim.x, tid = threadIdx.x, hl = nt >> 2;
    auto push = [&](size_t off, int hf, int t, int tn) {
      size_t bo, bytes;
      part(off, bo, bytes);
      const size_t base = c.stageOff + (size_t)hf * c.stageBytes + (size_t)rank * slotCap + bo;
      for (int i = 1; i < n; i++) {
        const int p = (rank + i) % n;
        groupCopy(c.ws[p] + base, send + (size_t)p * total + off + bo, bytes, t, tn);
      }
    };
    auto copyOut = [&](size_t off, int hf, int t, int tn) {
      size_t bo, bytes;
      part(off, bo, bytes);
      const size_t base = c.stageOff + (size_t)hf * c.stageBytes + bo;
      for (int i = 1; i < n; i++) {
        const int s = (rank + n - i) % n;
        groupCopy(recv + (size_t)s * total + off + bo, c.ws[rank] + base + (size_t)s * slotCap, bytes, t, tn);
      }
    };
    push(0, half, tid, nt);
    ctaBarrier(c, epoch);
    for (size_t off = 0; off < total; off += cap, half ^= 1) {
      const bool more = off + cap < total;
      if (more) {
        if (tid >= hl) push(off + cap, half ^ 1, tid - hl, nt - hl);
        else copyOut(off, half, tid, hl);
      } else {
        copyOut(off, half, tid, nt);
      }
      if (tid < hl || !more) {   // the rank's own block, piece by piece beside the copy-out
        size_t bo, bytes;
        part(off, bo, bytes);
        groupCopy(recv + (size_t)rank * total + off + bo, send + (size_t)rank * total + off + bo, bytes, tid, more ? hl : nt);
      }
      if (more) ctaBarrier(c, epoch);
    }
    if (threadIdx.x == 0) c.local->barEpoch[b] = epoch;
    stampEnd(c);
    return;
  }

  if constexpr (!NVLS) {
    if (a.kind == COLL_BROADCAST && !a.direct && n > 2 && total >= ((size_t)512 << 10)) {
      // Broadcast through staging by peer stores, every link carrying each byte once (scatter and forward): a lane's part
      // of a chunk is cut into n - 1 regions, one per non-root rank. The root stores region o only into its owner's staging
      // half; the owner forwards it into the same place of every other non-root rank's half and copies it to its own recv;
      // after the step's barrier everybody copies the regions it was forwarded. So the root sends a chunk once, a non-root
      // rank receives a chunk once and sends (n - 2) / (n - 1) of one: the line rate of one link direction, against
      // 1 / (n - 1) of it if the root stored everything itself. Software pipeline, one barrier per chunk: in step k the root
      // already stores chunk k + 1 into the other half, three quarters of a non-root CTA forward chunk k and the last
      // quarter copies out (its own region of chunk k, the forwarded regions of chunk k - 1). A region of a half is
      // written again two steps after it was last read, behind the barrier in between; the root's stores of chunk k + 1
      // touch only the owner's own region of the other half, which nobody reads in step k. Short messages and two ranks
      // take the plain push below (one barrier less, nothing to forward).
      const int m = n - 1, root = a.root, tid = threadIdx.x, nt = blockDim.x;
      const bool isRoot = rank == root;
      const int own = (rank - root - 1 + n) % n;   // this rank's region (non-root ranks only)
      // Where a region lies depends on the lane's capacity only, never on how full a chunk is (a short last chunk laid out
      // differently would let the root's stores of chunk k + 1 land on regions of chunk k - 1 that are still being copied out).
      const size_t laneCap = perLane << 4;
      auto region = [&](size_t bo, size_t bytes, int o, size_t& ro, size_t& rb) {
        const size_t sub = (((laneCap + m - 1) / m) + 15) & ~(size_t)15;
        const size_t lo = (size_t)o * sub < bytes ? (size_t)o * sub : bytes;
        const size_t hi = lo + sub < bytes ? lo + sub : bytes;
        ro = bo + lo;
        rb = hi - lo;
      };
      auto rootPush = [&](size_t off, int hf, int t, int tn) {
        size_t bo, bytes;
        part(off, bo, bytes);
        const size_t base = c.stageOff + (size_t)hf * c.stageBytes;
        for (int o = 0; o < m; o++) {
          size_t ro, rb;
          region(bo, bytes, o, ro, rb);
          groupCopy(c.ws[(root + 1 + o) % n] + base + ro, send + off + ro, rb, t, tn);
        }
      };
      const int hl = nt >> 2;
      if (isRoot) rootPush(0, half, tid, nt);
      ctaBarrier(c, epoch);
      size_t prevOff = 0;
      int prevHalf = half;
      bool havePrev = false;
      for (size_t off = 0; off < total; off += cap, half ^= 1) {
        const bool more = off + cap < total;
        size_t bo, bytes;
        part(off, bo, bytes);
        const size_t base = c.stageOff + (size_t)half * c.stageBytes;
        if (isRoot) {
          const bool selfCopy = recv != send;
          if (tid >= hl || !selfCopy) {
            if (more) rootPush(off + cap, half ^ 1, selfCopy ? tid - hl : tid, selfCopy ? nt - hl : nt);
          } else {
            groupCopy(recv + off + bo, send + off + bo, bytes, tid, hl);
          }
        } else {
          size_t ro, rb;
          region(bo, bytes, own, ro, rb);
          if (tid >= hl) {  // forward this rank's region of chunk k to the other non-root ranks
            for (int i = 1; i < n; i++) {
              const int p = (rank + i) % n;
              if (p == root) continue;
              groupCopy(c.ws[p] + base + ro, c.ws[rank] + base + ro, rb, tid - hl, nt - hl);
            }
          } else {          // copy out: own region of chunk k, forwarded regions of chunk k - 1
            groupCopy(recv + off + ro, c.ws[rank] + base + ro, rb, tid, hl);
            if (havePrev) {
              size_t pbo, pbytes;
              part(prevOff, pbo, pbytes);
              const size_t pbase = c.stageOff + (size_t)prevHalf * c.stageBytes;
              for (int o = 0; o < m; o++) {
                if (o == own) continue;
                size_t qo, qb;
                region(pbo, pbytes, o, qo, qb);
                groupCopy(recv + prevOff + qo, c.ws[rank] + pbase + qo, qb, tid, hl);
              }
            }
          }
        }
        ctaBarrier(c, epoch);
        prevOff = off;
        prevHalf = half;
        havePrev = true;
      }
      if (!isRoot && havePrev) {  // the forwarded regions of the last chunk
        size_t pbo, pbytes;
        part(prevOff, pbo, pbytes);
        const size_t pbase = c.stageOff + (size_t)prevHalf * c.stageBytes;
        for (int o = 0; o < m; o++) {
          if (o == own) continue;
          size_t qo, qb;
          region(pbo, pbytes, o, qo, qb);
          ctaCopy(recv + prevOff + qo, c.ws[rank] + pbase + qo, qb);
        }
      }
      if (threadIdx.x == 0) c.local->barEpoch[b] = epoch;
      stampEnd(c);
      return;
    }
  }

  for (size_t off = 0; off < total; off += cap, half ^= 1) {
    const size_t stageBase = c.stageOff + (size_t)half * c.stageBytes;
    size_t bo, bytes;  // byte offset of this CTA's part inside the chunk, and its length
    part(off, bo, bytes);

    if (isAG) {  // direct windows: pull straight from the peers' send buffers
      ctaBarrier(c, epoch);
      const int tid = threadIdx.x, warps = blockDim.x >> 5, peers = n - 1;
      if (bytes <= (size_t)(64u << 10) && warps >= peers && peers > 1) {
        const int per = warps / peers, w = tid >> 5;  // short parts: all peers in flight at once
        if (w < per * peers) {
          const int p = (rank + 1 + w / per) % n;
          groupCopy(recv + (size_t)p * total + off + bo, a.sendPeer[p] + off + bo, bytes, (w % per) * 32 + (tid & 31), per * 32);
        }
      } else {
        for (int i = 1; i < n; i++) {
          const int p = (rank + i) % n;
          ctaCopy(recv + (size_t)p * total + off + bo, a.sendPeer[p] + off + bo, bytes);
        }
      }
      if (recv + (size_t)rank * total != send) ctaCopy(recv + (size_t)rank * total + off + bo, send + off + bo, bytes);
      ctaBarrier(c, epoch);
    } else {  // Broadcast
      if (a.direct) {
        ctaBarrier(c, epoch);
        if (rank == a.root) {
          if constexpr (NVLS) {
            ctaCopyToMc(a.recvMc + off + bo, send + off + bo, bytes);
          } else {
            // A quarter of the threads make the root's own copy (local memory, several times faster than the link)
            // while the others store to the peers, instead of one after the other.
            const int nt = blockDim.x, tid = threadIdx.x;
            const int hl = (recv != send) ? nt >> 2 : 0;
            if (tid < hl) {
              groupCopy(recv + off + bo, send + off + bo, bytes, tid, hl);
            } else {
              for (int i = 1; i < n; i++) groupCopy(a.recvPeer[(rank + i) % n] + off + bo, send + off + bo, bytes, tid - hl, nt - hl);
            }
          }
        }
        ctaBarrier(c, epoch);
      } else {
        // The root pushes: one multicast store stream through the switch, or plain stores into every peer's staging
        // (stores run faster over NVLink than the loads of a pull: 690 against 613 GB/s between two GPUs). Each
        // receiver then copies out of its OWN staging half while the root fills the other one.
        if (rank == a.root) {
          if constexpr (NVLS) {
            ctaCopyToMc(c.wsMc + stageBase + bo, send + off + bo, bytes);
            if (recv != send) ctaCopy(recv + off + bo, send + off + bo, bytes);
          } else {
            const int nt = blockDim.x, tid = threadIdx.x;
            const int hl = (recv != send) ? nt >> 2 : 0;   // the root's own copy runs beside the stores to the peers
            if (tid < hl) {
              groupCopy(recv + off + bo, send + off + bo, bytes, tid, hl);
            } else {
              for (int i = 1; i < n; i++) groupCopy(c.ws[(rank + i) % n] + stageBase + bo, send + off + bo, bytes, tid - hl, nt - hl);
            }
          }
        }
        ctaBarrier(c, epoch);
        if (rank != a.root) ctaCopy(recv + off + bo, c.ws[rank] + stageBase + bo, bytes);
      }
    }
  }
  if (threadIdx.x == 0) c.local->barEpoch[b] = epoch;
  stampEnd(c);
}

// ---- grouped send/recv ----------------------------------------------------------------------
// Non-template kernels are compiled only by the translation unit that launches them.
#ifdef B200_MISC_KERNELS
// Flag-in-data all-gather: every rank stores its slice, 8 bytes of data and 8 of flags per line, into its slot of every
// peer's buffer; a receiver copies a line out as soon as both flags show this operation's number. No barrier, no
// staging round: one launch and one trip over the link. a.count is the slice in BYTES (the type does not matter).
// With a.kind == COLL_ALLTOALL every destination gets its own chunk of a.count bytes instead of the same slice.
__device__ __forceinline__ uint2 llLoad8(const char* base, size_t bytes, size_t i, bool aligned) {
  const size_t b0 = i * 8;
  if (aligned && b0 + 8 <= bytes) return *(const uint2*)(base + b0);
  union { uint2 v; unsigned char b[8]; } u;
  u.v = make_uint2(0, 0);
  for (int k = 0; k < 8; k++)
    if (b0 + k < bytes) u.b[k] = (unsigned char)base[b0 + k];
  return u.v;
}
__device__ __forceinline__ void llStore8(char* base, size_t bytes, size_t i, bool aligned, uint2 v) {
  const size_t b0 = i * 8;
  if (aligned && b0 + 8 <= bytes) { *(uint2*)(base + b0) = v; return; }
  union { uint2 v; unsigned char b[8]; } u;
  u.v = v;
  for (int k = 0; k < 8; k++)
    if (b0 + k < bytes) base[b0 + k] = (char)u.b[k];
}

__global__ void __launch_bounds__(kCollThreads) kLLAllGather(const __grid_constant__ DevComm c, const __grid_constant__ LLArgs a) {
  stampBegin(c);
  const int n = c.nranks, rank = c.rank;
  const size_t bytes = a.count;
  const size_t units = (bytes + 7) / 8;
  const size_t halfOff = kWsLLOff + (size_t)(a.seq & 1) * (size_t)n * c.llSlotBytes;
  const char* send = (const char*)a.send;
  char* recv = (char*)a.recv;
  const bool aligned = (((((uintptr_t)a.send) | ((uintptr_t)a.recv)) & 7) == 0) && (bytes % 8 == 0);
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t gn = (size_t)gridDim.x * blockDim.x;
  char* mine = recv + (size_t)rank * bytes;
  if (a.kind == COLL_ALLTOALL) {
    // The same exchange with a chunk of its own for every destination.
    for (size_t i = gtid; i < units; i += gn) {
      for (int d = 1; d < n; d++) {
        const int p = (rank + d) % n;
        const uint2 v = llLoad8(send + (size_t)p * bytes, bytes, i, aligned);
        stVolatile16(c.ws[p] + halfOff + (size_t)rank * c.llSlotBytes + i * 16, make_uint4(v.x, a.seq, v.y, a.seq));
      }
      llStore8(mine, bytes, i, aligned, llLoad8(send + (size_t)rank * bytes, bytes, i, aligned));
    }
  } else {
    const bool inPlace = mine == send;
    for (size_t i = gtid; i < units; i += gn) {
      const uint2 v = llLoad8(send, bytes, i, aligned);
      const uint4 line = make_uint4(v.x, a.seq, v.y, a.seq);
      for (int d = 1; d < n; d++) {
        const int p = (rank + d) % n;
        stVolatile16(c.ws[p] + halfOff + (size_t)rank * c.llSlotBytes + i * 16, line);
      }
      if (!inPlace) llStore8(mine, bytes, i, aligned, v);
    }
  }
  for (int d = 1; d < n; d++) {
    const int s = (rank + n - d) % n;
    char* dst = recv + (size_t)s * bytes;
    for (size_t i = gtid; i < units; i += gn) {
      const char* line = c.ws[rank] + halfOff + (size_t)s * c.llSlotBytes + i * 16;
      uint4 v;
      unsigned long long t0 = 0;
      uint32_t spins = 0;
      bool ok = true;
      while (true) {
        v = ldVolatile16(line);
        if (v.y == a.seq && v.w == a.seq) break;
        if ((++spins & 0xff) == 0) {
          if (*(volatile uint32_t*)&c.local->failed) { ok = false; break; }
          if (*c.abortFlag) { recordFailure(c, 2, WAIT_LL, s, a.seq, v.y); ok = false; break; }
          unsigned long long now = globalTimerNs();
          if (t0 == 0) t0 = now;
          else if (now - t0 > c.timeoutNs) { recordFailure(c, 1, WAIT_LL, s, a.seq, v.y); ok = false; break; }
        }
      }
      if (!ok) break;  // the failure is recorded; leave the rest of this source's lines
      llStore8(dst, bytes, i, aligned, make_uint2(v.x, v.z));
    }
  }
  stampEnd(c);
}

__global__ void __launch_bounds__(kCollThreads) kP2p(const __grid_constant__ DevComm c, const __grid_constant__ P2pArgs a) {
  stampBegin(c);
  const int subs = c.p2pSubs;
  const int w = blockIdx.x / subs, j = blockIdx.x % subs;
  if (w < a.nwork) {
    const P2pWork& wk = a.work[w];
    const int peer = wk.peer, rank = c.rank;
    size_t lo, hi;
    splitUnits((wk.bytes + 15) >> 4, subs, j, lo, hi);
    const size_t begin = lo << 4;
    const size_t end = (hi << 4) < wk.bytes ? (hi << 4) : wk.bytes;
    const size_t chunk = c.p2pChunkBytes;
    unsigned long long* myTail = (unsigned long long*)(c.ws[rank] + kWsP2pCtrlOff);
    unsigned long long* myHead = myTail + kMaxRanks * kMaxP2pSubs;
    unsigned long long* peerTail = (unsigned long long*)(c.ws[peer] + kWsP2pCtrlOff);
    unsigned long long* peerHead = peerTail + kMaxRanks * kMaxP2pSubs;
    __shared__ int okShared;
    if (wk.isSend) {
      unsigned long long sent = c.local->p2pSent[peer][j];
      char* fifo = c.ws[peer] + c.p2pOff + ((size_t)(rank * subs + j) * c.p2pSlots) * chunk;
      for (size_t o = begin; o < end; o += chunk) {
        const size_t nb = end - o < chunk ? end - o : chunk;
        if (threadIdx.x == 0) {
          unsigned long long need = sent + 1 > (unsigned long long)c.p2pSlots ? sent + 1 - c.p2pSlots : 0;
          okShared = waitGe64(c, &myHead[peer * kMaxP2pSubs + j], need, WAIT_P2P_CREDIT, peer) ? 1 : 0;
        }
        __syncthreads();
        if (okShared) ctaCopy(fifo + (size_t)(sent % c.p2pSlots) * chunk, wk.src + o, nb);
        __syncthreads();
        sent++;
        if (threadIdx.x == 0) {
          __threadfence_system();
          stReleaseSys64(&peerTail[rank * kMaxP2pSubs + j], sent);
        }
      }
      if (threadIdx.x == 0) c.local->p2pSent[peer][j] = sent;
    } else {
      unsigned long long recvd = c.local->p2pRecvd[peer][j];
      const char* fifo = c.ws[rank] + c.p2pOff + ((size_t)(peer * subs + j) * c.p2pSlots) * chunk;
      for (size_t o = begin; o < end; o += chunk) {
        const size_t nb = end - o < chunk ? end - o : chunk;
        if (threadIdx.x == 0) okShared = waitGe64(c, &myTail[peer * kMaxP2pSubs + j], recvd + 1, WAIT_P2P_DATA, peer) ? 1 : 0;
        __syncthreads();
        if (okShared) ctaCopy(wk.dst + o, fifo + (size_t)(recvd % c.p2pSlots) * chunk, nb);
        __syncthreads();
        recvd++;
        if (threadIdx.x == 0) {
          __threadfence_system();
          stReleaseSys64(&peerHead[rank * kMaxP2pSubs + j], recvd);
        }
      }
      if (threadIdx.x == 0) c.local->p2pRecvd[peer][j] = recvd;
    }
  }
  stampEnd(c);
}

// All-to-all by direct peer stores (the rccl-tests all-to-all moves count / nranks elements per peer pair in 16-byte
// aligned chunks, rccl-tests/src/alltoall.cpp:16-18, 67; here a chunk goes over NVLink once, with no FIFO in between).
// CTA b handles the same byte range of every chunk. Barrier before: every rank has entered the call, so its receive
// buffer may be overwritten. Barrier after: everything stored into this rank's buffer has landed.
__global__ void __launch_bounds__(kCollThreads) kAllToAllDirect(const __grid_constant__ DevComm c, const __grid_constant__ A2aDirectArgs a) {
  stampBegin(c);
  const int n = c.nranks, rank = c.rank;
  uint32_t epoch = c.local->barEpoch[blockIdx.x];
  size_t lo, hi;
  splitUnits(a.chunkBytes >> 4, gridDim.x, blockIdx.x, lo, hi);
  ctaBarrier(c, epoch);
  if (lo < hi) {
    for (int i = 0; i < n; i++) {
      const int p = (rank + i) % n;  // own chunk first (local), then the peers in ring order so that no two ranks start on the same target
      ctaCopy(a.recvPeer[p] + (size_t)rank * a.chunkBytes + (lo << 4), a.send + (size_t)p * a.chunkBytes + (lo << 4), (hi - lo) << 4);
    }
  }
  ctaBarrier(c, epoch);
  if (threadIdx.x == 0) c.local->barEpoch[blockIdx.x] = epoch;
  stampEnd(c);
}

__global__ void kBarrier(const __grid_constant__ DevComm c) {
  stampBegin(c);
  uint32_t epoch = c.local->barEpoch[0];
  ctaBarrier(c, epoch);
  if (threadIdx.x == 0) c.local->barEpoch[0] = epoch;
  stampEnd(c);
}
#endif  // B200_MISC_KERNELS

}  // namespace b200
