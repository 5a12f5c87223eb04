// Blackwell (sm_100a) building blocks in inline PTX: mbarriers with bounded waits, TMA tile loads
// (never with cluster multicast), tcgen05 tensor-memory allocation, UMMA descriptors, MMA issue,
// commit and accumulator loads. Used by the GEMM and the fused GEMM+collective kernels.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace b200 {
namespace sm100 {

__device__ __forceinline__ uint32_t smemAddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool electOne() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier ----------------------------------------------------------------------------------
__device__ __forceinline__ void mbarInit(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fenceBarrierInit() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fenceProxyAsync() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbarArrive(uint64_t* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ void mbarArriveExpectTx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbarTryWait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(smemAddr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll already blocks for a hardware-defined
// time slice), sets *err and returns false. Callers then drain and leave.
__device__ __forceinline__ bool mbarWait(uint64_t* bar, uint32_t parity, volatile int* err, int code, uint32_t limit = 4000000u) {
  for (uint32_t i = 0; i < limit; i++) {
    if (mbarTryWait(bar, parity)) return true;
    if ((i & 0x3ff) == 0x3ff && *err) return false;
  }
  atomicCAS((int*)err, 0, code);
  return false;
}

// ---- TMA ------------------------------------------------------------------------------------------
// 2-D tile load, global -> shared, completion counted in bytes on `bar`. x is the innermost
// coordinate (elements) and must keep x * sizeof(element) a multiple of 16 bytes.
__device__ __forceinline__ void tmaLoad2d(void* smemDst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smemAddr(smemDst)),
               "l"(map), "r"(x), "r"(y), "r"(smemAddr(bar))
               : "memory");
}
__device__ __forceinline__ void tmaStore2d(const CUtensorMap* map, const void* smemSrc, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(smemAddr(smemSrc)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tmaStoreCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tmaStoreWaitRead0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tmaStoreWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetchTensorMap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tensor memory -----------------------------------------------------------------------------------
// One whole warp allocates `cols` (power of two >= 32) columns; the base address lands in smem.
__device__ __forceinline__ void tmemAlloc(uint32_t* smemOut, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(smemOut)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmemRelinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmemDealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- UMMA descriptors -----------------------------------------------------------------------------------
// Shared-memory operand descriptor for a K-major tile whose rows are 128 bytes (64 bf16 / 128 fp8)
// laid out by TMA with the 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smemDescSw128(uint32_t smemByteAddr) {
  uint64_t d = 0;
  d |= (uint64_t)((smemByteAddr & 0x3ffff) >> 4);        // start address, 16-byte units
  d |= (uint64_t)0 << 16;                                // leading-dimension byte offset: unused for swizzled K-major
  d |= (uint64_t)(1024 >> 4) << 32;                      // stride between 8-row groups
  d |= (uint64_t)1 << 46;                                // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                                // layout: SWIZZLE_128B
  return d;
}
// Instruction descriptor: D fp32; A, B of the given format (kind::f16: 0 fp16, 1 bf16;
// kind::f8f6f4: 0 e4m3, 1 e5m2), both K-major, no negation, dense.
__host__ __device__ constexpr uint32_t instrDesc(uint32_t M, uint32_t N, uint32_t abFormat) {
  return (1u << 4) | (abFormat << 7) | (abFormat << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread.
__device__ __forceinline__ void mmaF16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmemD),
      "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mmaF8(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmemD),
      "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every MMA this thread issued so far has finished.
__device__ __forceinline__ void mmaCommit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smemAddr(bar)) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets row (lane base + t).
__device__ __forceinline__ void tmemLoad32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmemLoadWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- CTA pairs (cta_group::2) ---------------------------------------------------------------------------------
// Two CTAs of a cluster share one MMA: the even CTA of the pair issues it, each CTA holds half of the operands in its own
// shared memory and half of the accumulator rows in its own tensor memory. Loads are ordinary tile loads (one CTA's
// memory each, no multicast); what crosses the pair are mbarrier arrivals.
__device__ __forceinline__ uint32_t clusterCtaRank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `smemByteAddr` (an address in this CTA's shared memory) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapToCta(uint32_t smemByteAddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smemByteAddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void clusterArrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void clusterWait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void mbarArriveCluster(uint32_t clusterAddr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
// Tile load into THIS CTA's shared memory whose bytes are counted on a barrier of the pair's even CTA (`barClusterAddr`).
__device__ __forceinline__ void tmaLoad2dPair(void* smemDst, const CUtensorMap* map, int x, int y, uint32_t barClusterAddr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smemAddr(smemDst)),
               "l"(map), "r"(x), "r"(y), "r"(barClusterAddr)
               : "memory");
}
__device__ __forceinline__ void tmemAllocPair(uint32_t* smemOut, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(smemOut)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmemRelinquishPair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmemDeallocPair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mmaF16Pair(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmemD),
      "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at `barClusterAddr` (any CTA of the cluster) once every MMA this thread issued so far has finished.
__device__ __forceinline__ void mmaCommitPair(uint32_t barClusterAddr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(barClusterAddr) : "memory");
}
// The same arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair, with one instruction.
__device__ __forceinline__ void mmaCommitBoth(uint32_t barAddr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(barAddr), "h"((uint16_t)3) : "memory");
}

// Shared-memory operand descriptor for an MN-major tile laid out by TMA with the 128-byte swizzle: rows of 64 elements
// (128 bytes) along M or N, one row per step of the reduction dimension, 8 rows = one 1024-byte swizzle group; the next 64
// elements along M/N start `chunkBytes` further on (one TMA box).
__device__ __forceinline__ uint64_t smemDescSw128Mn(uint32_t smemByteAddr, uint32_t chunkBytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smemByteAddr & 0x3ffff) >> 4);
  d |= (uint64_t)((chunkBytes >> 4) & 0x3fff) << 16;      // leading-dimension byte offset: between 64-element chunks along M/N
  d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset: between groups of 8 reduction rows
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor with the operands' majors: 0 K-major, 1 MN-major.
__host__ __device__ constexpr uint32_t instrDescMajor(uint32_t M, uint32_t N, uint32_t abFormat, uint32_t aMn, uint32_t bMn) {
  return (1u << 4) | (abFormat << 7) | (abFormat << 10) | (aMn << 15) | (bMn << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

}  // namespace sm100
}  // namespace b200
