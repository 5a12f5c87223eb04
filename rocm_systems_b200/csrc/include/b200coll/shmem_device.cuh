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

// ---- barrier over all PEs -------------------------------------------------------------------------------------------
// Called by every thread of ONE block per PE (the same block index on every PE). Completes all of
// this block's earlier puts, then waits until every PE has arrived.
__device__ __forceinline__ int barrier_all_block(const b200shmem_dev_t& d) {
  __shared__ int result;
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned long long epoch = *d.syncEpoch + 1;
    __threadfence_system();
    for (int pe = 0; pe < d.npes; pe++) {
      unsigned long long* r = ptr(d, d.syncFlags, pe) + d.pe;
      asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(r), "l"(epoch) : "memory");
    }
    int rc = B200SHMEM_OK;
    for (int pe = 0; pe < d.npes && rc == B200SHMEM_OK; pe++) rc = signal_wait_until(d, d.syncFlags + pe, B200SHMEM_CMP_GE, epoch);
    *d.syncEpoch = epoch;
    result = rc;
  }
  __syncthreads();
  return result;
}
__device__ __forceinline__ int sync_all_block(const b200shmem_dev_t& d) { return barrier_all_block(d); }

}  // namespace b200shmem
