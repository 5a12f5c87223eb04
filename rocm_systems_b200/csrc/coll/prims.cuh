// Device primitives: system-scope flag stores/loads, bounded waits, the per-CTA inter-rank
// barrier, vector copies, and multimem (NVLS) loads/stores.
//
// Signals in the reference runtime are 64-bit values with acquire/release atomics and an abort
// timeout (rocr-runtime/runtime/hsa-runtime/core/runtime/default_signal.cpp:57-250,
// core/util/flag.h:265-267). Here a signal is a 32-bit epoch counter in peer-mapped memory; a
// waiter polls it with ld.acquire.sys and gives up after a %globaltimer budget, records why in
// DevStatus, and lets the kernel finish.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "device.h"

namespace b200 {

__device__ __forceinline__ uint32_t ldAcquireSys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ldAcquireSys64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void stReleaseSys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void stReleaseSys64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globalTimerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint4 ldStream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st16(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ldVolatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void stVolatile16(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- failure recording ---------------------------------------------------------------------
__device__ __forceinline__ void recordFailure(const DevComm& c, uint32_t code, uint32_t what, uint32_t peer,
                                              uint32_t expected, uint32_t seen) {
  if (atomicCAS(&c.local->failed, 0u, 1u) == 0u) {
    DevStatus* s = c.status;
    s->what = what;
    s->peer = peer;
    s->cta = blockIdx.x;
    s->expected = expected;
    s->seen = seen;
    s->opSeq = c.opSeq;
    __threadfence_system();
    s->code = code;
    __threadfence_system();
  }
}

// Spin until *flag >= target (wrap-safe), for at most c.timeoutNs. Returns false when the wait
// was given up; the caller keeps going (all addresses stay valid) and the kernel ends normally.
__device__ __forceinline__ bool waitGe(const DevComm& c, const uint32_t* flag, uint32_t target, uint32_t what, uint32_t peer) {
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  uint32_t v = 0;
  while (true) {
    v = ldAcquireSys(flag);
    if ((int32_t)(v - target) >= 0) return true;
    if ((++spins & 0xff) == 0) {
      if (*(volatile uint32_t*)&c.local->failed) return false;
      if (*c.abortFlag) { recordFailure(c, 2, what, peer, target, v); return false; }
      unsigned long long now = globalTimerNs();
      if (t0 == 0) t0 = now;
      else if (now - t0 > c.timeoutNs) { recordFailure(c, 1, what, peer, target, v); return false; }
      __nanosleep(64);
    }
  }
}
__device__ __forceinline__ bool waitGe64(const DevComm& c, const unsigned long long* flag, unsigned long long target,
                                         uint32_t what, uint32_t peer) {
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    unsigned long long v = ldAcquireSys64(flag);
    if (v >= target) return true;
    if ((++spins & 0xff) == 0) {
      if (*(volatile uint32_t*)&c.local->failed) return false;
      if (*c.abortFlag) { recordFailure(c, 2, what, peer, (uint32_t)target, (uint32_t)v); return false; }
      unsigned long long now = globalTimerNs();
      if (t0 == 0) t0 = now;
      else if (now - t0 > c.timeoutNs) { recordFailure(c, 1, what, peer, (uint32_t)target, (uint32_t)v); return false; }
      __nanosleep(64);
    }
  }
}

// ---- bulk asynchronous copies into shared memory --------------------------------------------
// cp.async.bulk (the untiled TMA copy, never with cluster multicast) brings a contiguous range of
// global memory, this GPU's or a peer's, into shared memory and counts the bytes on an mbarrier.
// What is in flight is bounded by shared memory instead of by registers, which is what lets one
// CTA per SM keep an NVLink direction busy. Both addresses and the size are multiples of 16.
__device__ __forceinline__ uint32_t smemU32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cmbarInit(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemU32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void cmbarExpectTx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smemU32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool cmbarTryWait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(smemU32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulkLoad(void* smemDst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smemU32(smemDst)), "l"(gsrc),
               "r"(bytes), "r"(smemU32(bar))
               : "memory");
}
// Wait for a phase of `bar` for at most c.timeoutNs; a wait that is given up is recorded like any
// other (the kernel keeps going on valid addresses and ends normally).
__device__ __forceinline__ bool cmbarWaitBounded(const DevComm& c, uint64_t* bar, uint32_t parity, uint32_t peer) {
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (cmbarTryWait(bar, parity)) return true;
    if ((++spins & 0x3f) == 0) {
      if (*(volatile uint32_t*)&c.local->failed) return false;
      if (*c.abortFlag) { recordFailure(c, 2, WAIT_BULK, peer, parity, 0); return false; }
      unsigned long long now = globalTimerNs();
      if (t0 == 0) t0 = now;
      else if (now - t0 > c.timeoutNs) { recordFailure(c, 1, WAIT_BULK, peer, parity, 0); return false; }
    }
  }
}

// ---- barrier between CTA `blockIdx.x` of every rank -----------------------------------------
// Everything this CTA wrote before the call is visible to the matching CTA of every rank after
// it. `epoch` is the CTA's running barrier count (loaded from LocalState at kernel entry).
__device__ __forceinline__ bool ctaBarrier(const DevComm& c, uint32_t& epoch) {
  __syncthreads();
  epoch++;
  bool ok = true;
  const int t = threadIdx.x;
  if (t < c.nranks) {
    __threadfence_system();
    uint32_t* remote = (uint32_t*)(c.ws[t] + kWsBarOff) + (size_t)blockIdx.x * kMaxRanks + c.rank;
    stReleaseSys(remote, epoch);
    const uint32_t* mine = (const uint32_t*)(c.ws[c.rank] + kWsBarOff) + (size_t)blockIdx.x * kMaxRanks + t;
    ok = waitGe(c, mine, epoch, WAIT_BARRIER, (uint32_t)t);
  }
  __syncthreads();
  return ok;
}

// ---- block ranges ---------------------------------------------------------------------------
// Split `units` 16-byte units over `parts` parts; part `i` gets [lo, hi).
__device__ __forceinline__ void splitUnits(size_t units, int parts, int i, size_t& lo, size_t& hi) {
  size_t per = (units + parts - 1) / parts;
  lo = per * (size_t)i;
  hi = lo + per;
  if (lo > units) lo = units;
  if (hi > units) hi = units;
}

// ---- copies ---------------------------------------------------------------------------------
// Copy `bytes` bytes with threads t = 0..nt-1 of a thread group (by default the whole CTA). Fast
// path when both ends are 16-byte aligned.
__device__ __forceinline__ void groupCopy(void* dst, const void* src, size_t bytes, const int t, const int nt) {
  if (bytes == 0) return;
  if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
    const size_t nvec = bytes >> 4;
    const uint4* s = (const uint4*)src;
    uint4* d = (uint4*)dst;
    size_t i = t;
    constexpr int U = 8;
    for (; i + (size_t)(U - 1) * nt < nvec; i += (size_t)U * nt) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; u++) v[u] = ldStream16(s + i + (size_t)u * nt);
#pragma unroll
      for (int u = 0; u < U; u++) st16(d + i + (size_t)u * nt, v[u]);
    }
    for (; i < nvec; i += nt) st16(d + i, ldStream16(s + i));
    const size_t done = nvec << 4;
    for (size_t b = done + t; b < bytes; b += nt) ((char*)dst)[b] = ((const char*)src)[b];
  } else if ((((uintptr_t)dst | (uintptr_t)src) & 3) == 0) {
    const size_t nw = bytes >> 2;
    const uint32_t* s = (const uint32_t*)src;
    uint32_t* d = (uint32_t*)dst;
    for (size_t i = t; i < nw; i += nt) d[i] = s[i];
    for (size_t b = (nw << 2) + t; b < bytes; b += nt) ((char*)dst)[b] = ((const char*)src)[b];
  } else {
    for (size_t b = t; b < bytes; b += nt) ((char*)dst)[b] = ((const char*)src)[b];
  }
}
__device__ __forceinline__ void ctaCopy(void* dst, const void* src, size_t bytes) { groupCopy(dst, src, bytes, threadIdx.x, blockDim.x); }

// ---- multimem (NVLS) ------------------------------------------------------------------------
// One 16-byte in-switch reduction over every rank's copy of `mcAddr`, and the matching
// multicast store. These are switch-side operations on a multicast address; they are not TMA.
template <typename T> struct McReduce;  // specialised for the types the switch can add
template <> struct McReduce<float> {
  static __device__ __forceinline__ uint4 ld(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
template <> struct McReduce<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
template <> struct McReduce<__half> {
  static __device__ __forceinline__ uint4 ld(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
__device__ __forceinline__ void mcStore16(void* p, uint4 v) {
  // A weak store: ordering comes from the fence and release store of the barrier that follows every store phase.
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- trace stamps ---------------------------------------------------------------------------
__device__ __forceinline__ void stampBegin(const DevComm& c) {
  if (c.stamp && threadIdx.x == 0) atomicMin(&c.stamp->begin, globalTimerNs());
}
__device__ __forceinline__ void stampEnd(const DevComm& c) {
  if (c.stamp && threadIdx.x == 0) atomicMax(&c.stamp->end, globalTimerNs());
}

}  // namespace b200
