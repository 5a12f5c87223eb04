// b200shmem device API: callable from any CUDA kernel that received a b200shmem_dev_t.
//
// Naming follows OpenSHMEM (put/get/p/g, put_signal, signal_wait_until, atomic_*, fence, quiet,
// barrier_all) with thread / warp / block scopes as suffixes. Remote addresses are formed from
// symmetric local addresses by b200shmem_ptr_d(); all traffic is plain loads/stores/atomics on
// peer-mapped memory over NVLink. Waits are bounded: they return B200SHMEM_TIMEOUT after the
// context's budget and record it in dev.status, the kernel is expected to wind down.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "b200coll/shmem.h"

namespace b200shmem {

template <typename T>
__device__ __forceinline__ T* ptr(const b200shmem_dev_t& d, const T* local, int pe) {
  const unsigned long long off = (unsigned long long)((const char*)local - d.heap[d.pe]);
  return (T*)(d.heap[pe] + off);
}
template <typename T>
__device__ __forceinline__ T* mcPtr(const b200shmem_dev_t& d, const T* local) {
  return d.heapMc ? (T*)(d.heapMc + ((const char*)local - d.heap[d.pe])) : (T*)nullptr;
}

// ---- ordering -------------------------------------------------------------------------------------
__device__ __forceinline__ void fence() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void quiet() { __threadfence_system(); }

// ---- single elements ------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ void p(const b200shmem_dev_t& d, T* dest, T value, int pe) { *(volatile T*)ptr(d, dest, pe) = value; }
template <typename T> __device__ __forceinline__ T g(const b200shmem_dev_t& d, const T* source, int pe) { return *(volatile const T*)ptr(d, source, pe); }

// ---- bulk put/get ------------------------------------------------------------------------------------
__device__ __forceinline__ void copyStrided(char* dst, const char* src, size_t bytes, int t, int nt) {
  if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
    const size_t nv = bytes >> 4;
    for (size_t i = t; i < nv; i += nt) {
      uint4 v;
      asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + (i << 4)) : "memory");
      asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst + (i << 4)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    }
    for (size_t b = (nv << 4) + t; b < bytes; b += nt) dst[b] = src[b];
  } else {
    for (size_t b = t; b < bytes; b += nt) dst[b] = src[b];
  }
}
__device__ __forceinline__ void putmem(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes, int pe) {
  copyStrided((char*)ptr(d, (char*)dest, pe), (const char*)source, bytes, 0, 1);
}
__device__ __forceinline__ void getmem(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes, int pe) {
  copyStrided((char*)dest, (const char*)ptr(d, (const char*)source, pe), bytes, 0, 1);
}
__device__ __forceinline__ void putmem_warp(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes, int pe) {
  copyStrided((char*)ptr(d, (char*)dest, pe), (const char*)source, bytes, threadIdx.x & 31, 32);
  __syncwarp();
}
__device__ __forceinline__ void getmem_warp(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes, int pe) {
  copyStrided((char*)dest, (const char*)ptr(d, (const char*)source, pe), bytes, threadIdx.x & 31, 32);
  __syncwarp();
}
__device__ __forceinline__ void putmem_block(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes, int pe) {
  copyStrided((char*)ptr(d, (char*)dest, pe), (const char*)source, bytes, threadIdx.x, blockDim.x);
  __syncthreads();
}
__device__ __forceinline__ void getmem_block(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes, int pe) {
  copyStrided((char*)dest, (const char*)ptr(d, (const char*)source, pe), bytes, threadIdx.x, blockDim.x);
  __syncthreads();
}

// ---- signals ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void signal_op(const b200shmem_dev_t& d, unsigned long long* sigAddr, unsigned long long signal, int sigOp, int pe) {
  unsigned long long* r = ptr(d, sigAddr, pe);
  if (sigOp == B200SHMEM_SIGNAL_ADD) asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(r), "l"(signal) : "memory");
  else asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(r), "l"(signal) : "memory");
}
// Data, then the signal, in that order as seen by the target (block scope: all threads call it).
__device__ __forceinline__ void putmem_signal_block(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes,
                                                    unsigned long long* sigAddr, unsigned long long signal, int sigOp, int pe) {
  copyStrided((char*)ptr(d, (char*)dest, pe), (const char*)source, bytes, threadIdx.x, blockDim.x);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    signal_op(d, sigAddr, signal, sigOp, pe);
  }
}
__device__ __forceinline__ unsigned long long signal_fetch(const unsigned long long* sigAddr) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(sigAddr) : "memory");
  return v;
}
__device__ __forceinline__ bool cmpOk(unsigned long long v, int cmp, unsigned long long ref) {
  switch (cmp) {
    case B200SHMEM_CMP_EQ: return v == ref;
    case B200SHMEM_CMP_NE: return v != ref;
    case B200SHMEM_CMP_GT: return v > ref;
    case B200SHMEM_CMP_GE: return v >= ref;
    case B200SHMEM_CMP_LT: return v < ref;
    default: return v <= ref;
  }
}
// Waits on a local signal word. Returns B200SHMEM_OK, or B200SHMEM_TIMEOUT once the budget is spent.
__device__ __forceinline__ int signal_wait_until(const b200shmem_dev_t& d, const unsigned long long* sigAddr, int cmp, unsigned long long value,
                                                 unsigned long long* seen = nullptr) {
  unsigned long long t0 = 0;
  unsigned spins = 0;
  while (true) {
    const unsigned long long v = signal_fetch(sigAddr);
    if (cmpOk(v, cmp, value)) {
      if (seen) *seen = v;
      return B200SHMEM_OK;
    }
    if ((++spins & 0xff) == 0) {
      if (*(volatile int*)d.status) return B200SHMEM_TIMEOUT;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > d.timeoutNs) {
        atomicCAS(d.status, 0, B200SHMEM_TIMEOUT);
        return B200SHMEM_TIMEOUT;
      }
      __nanosleep(64);
    }
  }
}

// ---- atomics on a remote word ---------------------------------------------------------------------------------
#define B200SHMEM_ATOMIC(NAME, PTXOP, T, PTXT, REG)                                                                   \
  __device__ __forceinline__ T atomic_fetch_##NAME(const b200shmem_dev_t& d, T* dest, T value, int pe) {                \
    T old;                                                                                                              \
    asm volatile("atom.acq_rel.sys.global." PTXOP "." PTXT " %0, [%1], %2;" : "=" REG(old) : "l"(ptr(d, dest, pe)), REG(value) : "memory"); \
    return old;                                                                                                         \
  }                                                                                                                     \
  __device__ __forceinline__ void atomic_##NAME(const b200shmem_dev_t& d, T* dest, T value, int pe) {                   \
    asm volatile("red.release.sys.global." PTXOP "." PTXT " [%0], %1;" ::"l"(ptr(d, dest, pe)), REG(value) : "memory"); \
  }
B200SHMEM_ATOMIC(add, "add", unsigned int, "u32", "r")
B200SHMEM_ATOMIC(add, "add", unsigned long long, "u64", "l")
B200SHMEM_ATOMIC(and, "and", unsigned int, "b32", "r")
B200SHMEM_ATOMIC(and, "and", unsigned long long, "b64", "l")
B200SHMEM_ATOMIC(or, "or", unsigned int, "b32", "r")
B200SHMEM_ATOMIC(or, "or", unsigned long long, "b64", "l")
B200SHMEM_ATOMIC(xor, "xor", unsigned int, "b32", "r")
B200SHMEM_ATOMIC(xor, "xor", unsigned long long, "b64", "l")
#undef B200SHMEM_ATOMIC

__device__ __forceinline__ unsigned int atomic_swap(const b200shmem_dev_t& d, unsigned int* dest, unsigned int value, int pe) {
  unsigned int old;
  asm volatile("atom.acq_rel.sys.global.exch.b32 %0, [%1], %2;" : "=r"(old) : "l"(ptr(d, dest, pe)), "r"(value) : "memory");
  return old;
}
__device__ __forceinline__ unsigned long long atomic_swap(const b200shmem_dev_t& d, unsigned long long* dest, unsigned long long value, int pe) {
  unsigned long long old;
  asm volatile("atom.acq_rel.sys.global.exch.b64 %0, [%1], %2;" : "=l"(old) : "l"(ptr(d, dest, pe)), "l"(value) : "memory");
  return old;
}
__device__ __forceinline__ unsigned int atomic_compare_swap(const b200shmem_dev_t& d, unsigned int* dest, unsigned int cond, unsigned int value, int pe) {
  unsigned int old;
  asm volatile("atom.acq_rel.sys.global.cas.b32 %0, [%1], %2, %3;" : "=r"(old) : "l"(ptr(d, dest, pe)), "r"(cond), "r"(value) : "memory");
  return old;
}
__device__ __forceinline__ unsigned long long atomic_compare_swap(const b200shmem_dev_t& d, unsigned long long* dest, unsigned long long cond,
                                                                  unsigned long long value, int pe) {
  unsigned long long old;
  asm volatile("atom.acq_rel.sys.global.cas.b64 %0, [%1], %2, %3;" : "=l"(old) : "l"(ptr(d, dest, pe)), "l"(cond), "l"(value) : "memory");
  return old;
}
template <typename T> __device__ __forceinline__ T atomic_fetch(const b200shmem_dev_t& d, const T* source, int pe) {
  return atomic_fetch_add(d, const_cast<T*>(source), (T)0, pe);
}
template <typename T> __device__ __forceinline__ void atomic_set(const b200shmem_dev_t& d, T* dest, T value, int pe) { (void)atomic_swap(d, dest, value, pe); }

// ---- teams and barriers --------------------------------------------------------------------------------------------------
// A team is the PEs start, start + stride, ...; member i is PE start + i * stride. The world team shares barrier_all's words.
__device__ __forceinline__ b200shmem_team_t team_world(const b200shmem_dev_t& d) { return b200shmem_team_t{0, 1, d.npes, d.pe, d.syncFlags, d.syncEpoch}; }
__device__ __forceinline__ int team_my_pe(const b200shmem_team_t& t) { return t.idx; }
__device__ __forceinline__ int team_n_pes(const b200shmem_team_t& t) { return t.size; }
__device__ __forceinline__ int team_pe(const b200shmem_team_t& t, int idx) { return t.start + idx * t.stride; }   // number in the world
__device__ __forceinline__ int team_translate_pe(const b200shmem_team_t& src, int idx, const b200shmem_team_t& dst) {
  if (idx < 0 || idx >= src.size) return -1;
  const int off = team_pe(src, idx) - dst.start;
  if (off < 0 || off % dst.stride) return -1;
  return off / dst.stride < dst.size ? off / dst.stride : -1;
}

// Called by every thread of ONE block per member PE (the same block index on every PE). Completes all of this block's
// earlier puts, then waits until every member has arrived. Teams have their own arrival words and count their own
// barriers, so disjoint teams (and a team and its parent, used alternately) do not disturb one another.
__device__ __forceinline__ int team_sync_block(const b200shmem_dev_t& d, const b200shmem_team_t& t) {
  __shared__ int result;
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned long long epoch = *t.syncEpoch + 1;
    __threadfence_system();
    for (int i = 0; i < t.size; i++) {
      unsigned long long* r = ptr(d, t.syncFlags, team_pe(t, i)) + t.idx;
      asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(r), "l"(epoch) : "memory");
    }
    int rc = B200SHMEM_OK;
    for (int i = 0; i < t.size && rc == B200SHMEM_OK; i++) rc = signal_wait_until(d, t.syncFlags + i, B200SHMEM_CMP_GE, epoch);
    *t.syncEpoch = epoch;
    result = rc;
  }
  __syncthreads();
  return result;
}
__device__ __forceinline__ int barrier_all_block(const b200shmem_dev_t& d) { return team_sync_block(d, team_world(d)); }
__device__ __forceinline__ int sync_all_block(const b200shmem_dev_t& d) { return barrier_all_block(d); }

// ---- identity -------------------------------------------------------------------------------------------------------
__device__ __forceinline__ int my_pe(const b200shmem_dev_t& d) { return d.pe; }
__device__ __forceinline__ int n_pes(const b200shmem_dev_t& d) { return d.npes; }

// ---- point-to-point synchronisation on ordinary symmetric words (OpenSHMEM wait_until / test and their vector forms) -------
// T: a 32- or 64-bit integer type. The word is local; a peer changes it with p(), a put or an atomic.
template <typename T> __device__ __forceinline__ T load_acquire(const T* ivar) {
  static_assert(sizeof(T) == 4 || sizeof(T) == 8, "wait_until / test work on 32- and 64-bit words");
  if constexpr (sizeof(T) == 8) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(ivar) : "memory");
    return (T)v;
  } else {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ivar) : "memory");
    return (T)v;
  }
}
template <typename T> __device__ __forceinline__ bool cmpOkT(T v, int cmp, T ref) {
  switch (cmp) {
    case B200SHMEM_CMP_EQ: return v == ref;
    case B200SHMEM_CMP_NE: return v != ref;
    case B200SHMEM_CMP_GT: return v > ref;
    case B200SHMEM_CMP_GE: return v >= ref;
    case B200SHMEM_CMP_LT: return v < ref;
    default: return v <= ref;
  }
}
template <typename T> __device__ __forceinline__ bool test(const T* ivar, int cmp, T value) { return cmpOkT(load_acquire(ivar), cmp, value); }
// Index of the first of ivars[0..n) that satisfies the comparison, or -1 (one pass, no waiting): test_any.
template <typename T> __device__ __forceinline__ int test_any(const T* ivars, int n, int cmp, T value) {
  for (int i = 0; i < n; i++)
    if (test(ivars + i, cmp, value)) return i;
  return -1;
}
// Bounded like every wait: B200SHMEM_OK, or B200SHMEM_TIMEOUT once the context's time limit is spent (recorded in d.status).
template <typename T> __device__ __forceinline__ int wait_until(const b200shmem_dev_t& d, const T* ivar, int cmp, T value) {
  unsigned long long t0 = 0;
  unsigned spins = 0;
  while (true) {
    if (test(ivar, cmp, value)) return B200SHMEM_OK;
    if ((++spins & 0xff) == 0) {
      if (*(volatile int*)d.status) return B200SHMEM_TIMEOUT;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > d.timeoutNs) {
        atomicCAS(d.status, 0, B200SHMEM_TIMEOUT);
        return B200SHMEM_TIMEOUT;
      }
      __nanosleep(64);
    }
  }
}
template <typename T> __device__ __forceinline__ int wait_until_all(const b200shmem_dev_t& d, const T* ivars, int n, int cmp, T value) {
  for (int i = 0; i < n; i++)
    if (wait_until(d, ivars + i, cmp, value) != B200SHMEM_OK) return B200SHMEM_TIMEOUT;
  return B200SHMEM_OK;
}
// Waits until one of ivars[0..n) satisfies the comparison and stores its index in *which.
template <typename T> __device__ __forceinline__ int wait_until_any(const b200shmem_dev_t& d, const T* ivars, int n, int cmp, T value, int* which) {
  unsigned long long t0 = 0;
  unsigned spins = 0;
  while (true) {
    const int i = test_any(ivars, n, cmp, value);
    if (i >= 0) { *which = i; return B200SHMEM_OK; }
    if ((++spins & 0x3f) == 0) {
      if (*(volatile int*)d.status) return B200SHMEM_TIMEOUT;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > d.timeoutNs) {
        atomicCAS(d.status, 0, B200SHMEM_TIMEOUT);
        return B200SHMEM_TIMEOUT;
      }
      __nanosleep(64);
    }
  }
}

// ---- strided and non-blocking transfers --------------------------------------------------------------------------------------
// iput / iget: nelems elements, dest advancing by dst elements and source by sst elements per element (one thread).
template <typename T> __device__ __forceinline__ void iput(const b200shmem_dev_t& d, T* dest, const T* source, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, int pe) {
  T* r = ptr(d, dest, pe);
  for (size_t i = 0; i < nelems; i++) r[(ptrdiff_t)i * dst] = source[(ptrdiff_t)i * sst];
}
template <typename T> __device__ __forceinline__ void iget(const b200shmem_dev_t& d, T* dest, const T* source, ptrdiff_t dst, ptrdiff_t sst, size_t nelems, int pe) {
  const T* r = ptr(d, source, pe);
  for (size_t i = 0; i < nelems; i++) dest[(ptrdiff_t)i * dst] = r[(ptrdiff_t)i * sst];
}
// Stores to a peer are posted (the thread does not wait for them) and become visible at the latest at quiet(), a fence
// or a barrier, so the non-blocking put is the put; a get has returned its data when the call returns.
__device__ __forceinline__ void putmem_nbi(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes, int pe) { putmem(d, dest, source, bytes, pe); }
__device__ __forceinline__ void getmem_nbi(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes, int pe) { getmem(d, dest, source, bytes, pe); }
__device__ __forceinline__ void putmem_nbi_block(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes, int pe) { putmem_block(d, dest, source, bytes, pe); }
__device__ __forceinline__ void getmem_nbi_block(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes, int pe) { getmem_block(d, dest, source, bytes, pe); }

// ---- collectives of one block per PE -------------------------------------------------------------------------------------------
// Like barrier_all_block these are called by every thread of ONE block per PE, by all PEs, with symmetric dest / source.
// The pushing ones (broadcast, fcollect, alltoall) require, as OpenSHMEM does, that dest is free to be written on every PE
// at entry; they return after a barrier, when every PE's dest is complete. All return B200SHMEM_OK or B200SHMEM_TIMEOUT.
//
// Every collective exists in two forms: over a team (member indices wherever a PE is named: `root`, the block order of
// fcollect / alltoall) and over all PEs.
//
// dest on every member (the root's too, unless dest == source there) = the root's source.
__device__ __forceinline__ int broadcastmem_block(const b200shmem_dev_t& d, const b200shmem_team_t& t, void* dest, const void* source, size_t bytes, int root) {
  if (t.idx == root) {
    for (int i = 1; i < t.size; i++) putmem_block(d, dest, source, bytes, team_pe(t, (root + i) % t.size));
    if (dest != source) putmem_block(d, dest, source, bytes, team_pe(t, root));
  }
  return team_sync_block(d, t);
}
// dest [size][bytes] on every member: block i is member i's source (all-gather; OpenSHMEM fcollect).
__device__ __forceinline__ int fcollectmem_block(const b200shmem_dev_t& d, const b200shmem_team_t& t, void* dest, const void* source, size_t bytes) {
  for (int i = 0; i < t.size; i++) putmem_block(d, (char*)dest + (size_t)t.idx * bytes, source, bytes, team_pe(t, (t.idx + i) % t.size));
  return team_sync_block(d, t);
}
// source [size][bytes], dest [size][bytes]: block i of this member's source becomes block my-index of member i's dest.
__device__ __forceinline__ int alltoallmem_block(const b200shmem_dev_t& d, const b200shmem_team_t& t, void* dest, const void* source, size_t bytes) {
  for (int i = 0; i < t.size; i++) {
    const int m = (t.idx + i) % t.size;
    putmem_block(d, (char*)dest + (size_t)t.idx * bytes, (const char*)source + (size_t)m * bytes, bytes, team_pe(t, m));
  }
  return team_sync_block(d, t);
}
struct SumOp { template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a + b; } };
struct MaxOp { template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a > b ? a : b; } };
struct MinOp { template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a < b ? a : b; } };
// dest[i] = op over the team's members of source[i] on every member (OpenSHMEM *_reduce / *_to_all). Two steps: member m
// folds slice m of every member's source in member order 0, 1, ... into slice m of its own dest; then every member fetches
// the other slices from their owners. Each element is reduced exactly once, so the result is bit-identical everywhere, and
// dest may be source: slice m of member m is read by nobody but member m in the first step, and the other slices are
// overwritten only after the barrier that ends it. Barriers: before (all sources are written), between, and after (nobody
// reads this member's dest any more).
template <typename T, typename Op>
__device__ __forceinline__ int reduce_block(const b200shmem_dev_t& d, const b200shmem_team_t& t, T* dest, const T* source, size_t nreduce, Op op) {
  int rc = team_sync_block(d, t);
  if (rc != B200SHMEM_OK) return rc;
  const size_t per = (nreduce + t.size - 1) / t.size;
  const size_t lo = per * t.idx < nreduce ? per * t.idx : nreduce;
  const size_t hi = lo + per < nreduce ? lo + per : nreduce;
  for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    T acc = *(volatile const T*)(ptr(d, source, team_pe(t, 0)) + i);
    for (int m = 1; m < t.size; m++) acc = op(acc, (T) * (volatile const T*)(ptr(d, source, team_pe(t, m)) + i));
    dest[i] = acc;
  }
  rc = team_sync_block(d, t);
  if (rc != B200SHMEM_OK) return rc;
  for (int k = 1; k < t.size; k++) {
    const int q = (t.idx + k) % t.size;
    const size_t qlo = per * q < nreduce ? per * q : nreduce;
    const size_t qhi = qlo + per < nreduce ? qlo + per : nreduce;
    if (qhi > qlo) getmem_block(d, dest + qlo, dest + qlo, (qhi - qlo) * sizeof(T), team_pe(t, q));
  }
  return team_sync_block(d, t);
}
template <typename T> __device__ __forceinline__ int sum_reduce_block(const b200shmem_dev_t& d, const b200shmem_team_t& t, T* dest, const T* source, size_t n) { return reduce_block(d, t, dest, source, n, SumOp{}); }
template <typename T> __device__ __forceinline__ int max_reduce_block(const b200shmem_dev_t& d, const b200shmem_team_t& t, T* dest, const T* source, size_t n) { return reduce_block(d, t, dest, source, n, MaxOp{}); }
template <typename T> __device__ __forceinline__ int min_reduce_block(const b200shmem_dev_t& d, const b200shmem_team_t& t, T* dest, const T* source, size_t n) { return reduce_block(d, t, dest, source, n, MinOp{}); }

// The same over all PEs.
__device__ __forceinline__ int broadcastmem_block(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes, int root) { return broadcastmem_block(d, team_world(d), dest, source, bytes, root); }
__device__ __forceinline__ int fcollectmem_block(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes) { return fcollectmem_block(d, team_world(d), dest, source, bytes); }
__device__ __forceinline__ int alltoallmem_block(const b200shmem_dev_t& d, void* dest, const void* source, size_t bytes) { return alltoallmem_block(d, team_world(d), dest, source, bytes); }
template <typename T, typename Op>
__device__ __forceinline__ int reduce_block(const b200shmem_dev_t& d, T* dest, const T* source, size_t nreduce, Op op) { return reduce_block(d, team_world(d), dest, source, nreduce, op); }
template <typename T> __device__ __forceinline__ int sum_reduce_block(const b200shmem_dev_t& d, T* dest, const T* source, size_t n) { return reduce_block(d, dest, source, n, SumOp{}); }
template <typename T> __device__ __forceinline__ int max_reduce_block(const b200shmem_dev_t& d, T* dest, const T* source, size_t n) { return reduce_block(d, dest, source, n, MaxOp{}); }
template <typename T> __device__ __forceinline__ int min_reduce_block(const b200shmem_dev_t& d, T* dest, const T* source, size_t n) { return reduce_block(d, dest, source, n, MinOp{}); }

}  // namespace b200shmem
