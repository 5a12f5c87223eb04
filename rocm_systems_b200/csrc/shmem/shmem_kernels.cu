// b200shmem host API and the kernels behind its stream-ordered operations and self-tests.
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "../coll/launch.h"
#include "../core/comm.h"
#include "b200coll/shmem.h"
#include "b200coll/shmem_device.cuh"

using namespace b200;

struct b200shmem_ctx {
  Comm* comm = nullptr;
  char* heap = nullptr;          // local base of the symmetric window
  size_t heapBytes = 0;
  b200shmem_dev_t dev{};
  void* devState = nullptr;      // syncEpoch (u64) + status (int) + one barrier count per team slot, in local device memory
  int teamSlots = 1;             // slots of the heap's reserved head handed out so far (slot 0: all PEs)
  std::mutex mu;
  std::map<size_t, size_t> freeList;   // offset -> size
  std::map<size_t, size_t> live;       // offset -> size
  // Copy-engine transfers: side streams a large copy is split over, created on first use.
  cudaStream_t dmaStream[B200SHMEM_MAX_DMA_GANG] = {};
  cudaEvent_t dmaFork = nullptr, dmaJoin[B200SHMEM_MAX_DMA_GANG] = {};
  int dmaReady = 0;
};

namespace {

constexpr size_t kReserved = 4096;  // head of the heap: barrier arrival words, 64 bytes (8 PEs) per team slot
constexpr size_t kDevStateBytes = 64 + 8 * B200SHMEM_MAX_TEAMS;   // epoch, status, then one epoch per team slot
static_assert(kReserved >= 64 * B200SHMEM_MAX_TEAMS, "one 64-byte slot of arrival words per team");
constexpr size_t kAlign = 256;

__global__ void kSignal(b200shmem_dev_t d, unsigned long long* sig, unsigned long long value, int op, int pe) {
  if (threadIdx.x == 0) {
    __threadfence_system();
    b200shmem::signal_op(d, sig, value, op, pe);
  }
}
__global__ void kSignalWait(b200shmem_dev_t d, const unsigned long long* sig, int cmp, unsigned long long value) {
  if (threadIdx.x == 0) b200shmem::signal_wait_until(d, sig, cmp, value);
}
__global__ void kBarrierAll(b200shmem_dev_t d) { b200shmem::barrier_all_block(d); }

// Ring exchange driven entirely from the device: put+signal to the right neighbour, wait for
// the left neighbour's signal, verify, barrier, repeat.
__device__ __forceinline__ void ringBody(const b200shmem_dev_t& d, unsigned long long* data /*[2][count]*/, unsigned long long* src,
                                         unsigned long long* sig /*[2]*/, size_t count, int rounds, int* errors) {
  const int right = (d.pe + 1) % d.npes, left = (d.pe + d.npes - 1) % d.npes;
  int bad = 0;
  for (int r = 0; r < rounds; r++) {
    unsigned long long* slot = data + (size_t)(r & 1) * count;
    for (size_t i = threadIdx.x; i < count; i += blockDim.x) src[i] = (unsigned long long)d.pe * 1000003ull + (unsigned long long)r * 7ull + i;
    __syncthreads();
    b200shmem::putmem_signal_block(d, slot, src, count * sizeof(unsigned long long), sig + (r & 1), (unsigned long long)(r + 1), B200SHMEM_SIGNAL_SET, right);
    __shared__ int rc;
    if (threadIdx.x == 0) rc = b200shmem::signal_wait_until(d, sig + (r & 1), B200SHMEM_CMP_GE, (unsigned long long)(r + 1));
    __syncthreads();
    if (rc != B200SHMEM_OK) { bad++; break; }
    for (size_t i = threadIdx.x; i < count; i += blockDim.x)
      if (slot[i] != (unsigned long long)left * 1000003ull + (unsigned long long)r * 7ull + i) bad++;
    if (b200shmem::barrier_all_block(d) != B200SHMEM_OK) { bad++; break; }
  }
  if (bad) atomicAdd(errors, bad);
}

__global__ void kSelftestRing(b200shmem_dev_t d, unsigned long long* data, unsigned long long* src, unsigned long long* sig, size_t count, int rounds,
                              int* errors) {
  ringBody(d, data, src, sig, count, rounds, errors);
}

// words (on PE 0): [0] u64 counter (fetch_add), [1] u64 bit set (or), [2] u64 CAS counter,
// [3] u64 xor accumulator, [4] u32 counter, [5] u64 swap slot, [6] u64 and-mask.
__device__ __forceinline__ void atomicsBody(const b200shmem_dev_t& d, unsigned long long* words, int iters, int* errors) {
  int bad = 0;
  if (threadIdx.x == 0) {
    if (d.pe == 0) words[6] = ~0ull;
  }
  if (b200shmem::barrier_all_block(d) != B200SHMEM_OK) bad++;
  if (threadIdx.x == 0) {
    unsigned long long prev = 0;
    for (int i = 0; i < iters; i++) {
      unsigned long long old = b200shmem::atomic_fetch_add(d, &words[0], 1ull, 0);
      if (i > 0 && old <= prev) bad++;  // a fetch-add sequence seen by one PE is strictly increasing
      prev = old;
      b200shmem::atomic_add(d, (unsigned int*)&words[4], 1u, 0);
      // CAS increment
      unsigned long long cur = b200shmem::atomic_fetch(d, &words[2], 0);
      for (int tries = 0; tries < 100000; tries++) {
        unsigned long long seen = b200shmem::atomic_compare_swap(d, &words[2], cur, cur + 1, 0);
        if (seen == cur) break;
        cur = seen;
      }
      b200shmem::atomic_xor(d, &words[3], 1ull << d.pe, 0);
    }
    b200shmem::atomic_or(d, &words[1], 1ull << d.pe, 0);
    b200shmem::atomic_and(d, &words[6], ~(1ull << (d.pe + 32)), 0);
    (void)b200shmem::atomic_swap(d, &words[5], (unsigned long long)(d.pe + 1), 0);
  }
  if (b200shmem::barrier_all_block(d) != B200SHMEM_OK) bad++;
  if (threadIdx.x == 0) {
    const unsigned long long n = (unsigned long long)d.npes, it = (unsigned long long)iters;
    if (b200shmem::g(d, &words[0], 0) != n * it) bad++;
    if (b200shmem::g(d, &words[1], 0) != (1ull << d.npes) - 1) bad++;
    if (b200shmem::g(d, &words[2], 0) != n * it) bad++;
    if (b200shmem::g(d, &words[3], 0) != ((iters & 1) ? (1ull << d.npes) - 1 : 0ull)) bad++;
    if (b200shmem::g(d, (unsigned int*)&words[4], 0) != (unsigned int)(n * it)) bad++;
    const unsigned long long sw = b200shmem::g(d, &words[5], 0);
    if (sw < 1 || sw > n) bad++;
    unsigned long long mask = ~0ull;
    for (int pe = 0; pe < d.npes; pe++) mask &= ~(1ull << (pe + 32));
    if (b200shmem::g(d, &words[6], 0) != mask) bad++;
  }
  if (b200shmem::barrier_all_block(d) != B200SHMEM_OK) bad++;
  if (bad && threadIdx.x == 0) atomicAdd(errors, bad);
}

__global__ void kSelftestAtomics(b200shmem_dev_t d, unsigned long long* words, int iters, int* errors) { atomicsBody(d, words, iters, errors); }

// The block-scope collectives, the wait_until / test family and the strided put, each against its closed form.
// buf (symmetric, zeroed): A [npes * cnt] | B [npes * cnt] | R [cnt] | F [8] 64-bit words. One block per PE.
__device__ __forceinline__ void collBody(const b200shmem_dev_t& d, unsigned long long* buf, size_t cnt, int* errors) {
  using u64 = unsigned long long;
  const int n = d.npes, me = d.pe, right = (me + 1) % n, left = (me + n - 1) % n;
  u64* A = buf;
  u64* B = A + (size_t)n * cnt;
  u64* R = B + (size_t)n * cnt;
  u64* F = R + cnt;
  int bad = 0;
  const int root = 1 % n;
  // broadcast
  for (size_t i = threadIdx.x; i < cnt; i += blockDim.x) A[i] = (u64)me * 131 + i;
  __syncthreads();
  if (b200shmem::broadcastmem_block(d, B, A, cnt * 8, root) != B200SHMEM_OK) bad++;
  for (size_t i = threadIdx.x; i < cnt; i += blockDim.x)
    if (B[i] != (u64)root * 131 + i) bad++;
  if (b200shmem::barrier_all_block(d) != B200SHMEM_OK) bad++;  // everyone has checked B before it is written again
  // fcollect
  if (b200shmem::fcollectmem_block(d, B, A, cnt * 8) != B200SHMEM_OK) bad++;
  for (size_t i = threadIdx.x; i < (size_t)n * cnt; i += blockDim.x)
    if (B[i] != (u64)(i / cnt) * 131 + i % cnt) bad++;
  if (b200shmem::barrier_all_block(d) != B200SHMEM_OK) bad++;
  // alltoall
  for (size_t i = threadIdx.x; i < (size_t)n * cnt; i += blockDim.x) A[i] = (u64)me * 100000 + (u64)(i / cnt) * 1000 + i % cnt;
  __syncthreads();
  if (b200shmem::alltoallmem_block(d, B, A, cnt * 8) != B200SHMEM_OK) bad++;
  for (size_t i = threadIdx.x; i < (size_t)n * cnt; i += blockDim.x)
    if (B[i] != (u64)(i / cnt) * 100000 + (u64)me * 1000 + i % cnt) bad++;
  // reductions: sum in place, max out of place
  for (size_t i = threadIdx.x; i < cnt; i += blockDim.x) R[i] = (u64)me + i;
  __syncthreads();
  if (b200shmem::sum_reduce_block(d, R, R, cnt) != B200SHMEM_OK) bad++;
  for (size_t i = threadIdx.x; i < cnt; i += blockDim.x)
    if (R[i] != (u64)n * i + (u64)n * (n - 1) / 2) bad++;
  for (size_t i = threadIdx.x; i < cnt; i += blockDim.x) A[i] = (u64)((me * 7 + i) % 13);
  __syncthreads();
  if (b200shmem::max_reduce_block(d, B, A, cnt) != B200SHMEM_OK) bad++;
  for (size_t i = threadIdx.x; i < cnt; i += blockDim.x) {
    u64 m = 0;
    for (int pe = 0; pe < n; pe++) m = max(m, (u64)((pe * 7 + i) % 13));
    if (B[i] != m) bad++;
  }
  if (b200shmem::barrier_all_block(d) != B200SHMEM_OK) bad++;
  // strided put to the right neighbour (every second word of A there), then a flag word it waits on
  if (threadIdx.x == 0) {
    for (size_t i = 0; i < cnt; i++) R[i] = (u64)me * 17 + i + 1;
    b200shmem::iput(d, A, R, 2, 1, cnt / 2, right);
    b200shmem::fence();
    b200shmem::p(d, F + 1, (u64)(me + 1), right);
    if (b200shmem::wait_until(d, F + 1, B200SHMEM_CMP_EQ, (u64)(left + 1)) != B200SHMEM_OK) bad++;
    if (!b200shmem::test(F + 1, B200SHMEM_CMP_GE, (u64)1) || b200shmem::test(F + 2, B200SHMEM_CMP_NE, (u64)0)) bad++;
    int which = -1;
    if (b200shmem::wait_until_any(d, F, 4, B200SHMEM_CMP_NE, (u64)0, &which) != B200SHMEM_OK || which != 1) bad++;
    for (size_t i = 0; i < cnt / 2; i++)
      if (A[2 * i] != (u64)left * 17 + i + 1) bad++;
    if (b200shmem::my_pe(d) != me || b200shmem::n_pes(d) != n) bad++;
  }
  if (b200shmem::barrier_all_block(d) != B200SHMEM_OK) bad++;
  if (bad) atomicAdd(errors, bad);
}
__global__ void kSelftestColl(b200shmem_dev_t d, unsigned long long* buf, size_t cnt, int* errors) { collBody(d, buf, cnt, errors); }

// Collectives inside teams, every team at the same time as the others: `mine` is the team of this PE's parity, `sub` every
// second member of the even team (idx < 0 where this PE is not in it). Same buffer layout as above.
__device__ __forceinline__ void teamsBody(const b200shmem_dev_t& d, const b200shmem_team_t& mine, const b200shmem_team_t& sub, unsigned long long* buf,
                                          size_t cnt, int* errors) {
  using u64 = unsigned long long;
  namespace sh = b200shmem;
  const int n = d.npes, me = d.pe, ts = mine.size, ti = mine.idx;
  u64* A = buf;
  u64* B = A + (size_t)n * cnt;
  u64* R = B + (size_t)n * cnt;
  int bad = 0;
  if (sh::team_my_pe(mine) != ti || sh::team_n_pes(mine) != ts || sh::team_pe(mine, ti) != me) bad++;
  if (sh::team_translate_pe(mine, ti, sh::team_world(d)) != me || sh::team_translate_pe(sh::team_world(d), me, mine) != ti) bad++;
  const int nb = (me + 1) % n;   // a neighbour of the other parity is in no team of this one's
  if (((nb ^ me) & 1) && sh::team_translate_pe(sh::team_world(d), nb, mine) != -1) bad++;
  if (sh::team_sync_block(d, mine) != B200SHMEM_OK) bad++;
  const int root = ts - 1;
  for (size_t i = threadIdx.x; i < cnt; i += blockDim.x) A[i] = (u64)me * 131 + i;
  __syncthreads();
  if (sh::broadcastmem_block(d, mine, B, A, cnt * 8, root) != B200SHMEM_OK) bad++;
  for (size_t i = threadIdx.x; i < cnt; i += blockDim.x)
    if (B[i] != (u64)sh::team_pe(mine, root) * 131 + i) bad++;
  if (sh::barrier_all_block(d) != B200SHMEM_OK) bad++;   // a barrier of all PEs between two team collectives: separate counters
  if (sh::fcollectmem_block(d, mine, B, A, cnt * 8) != B200SHMEM_OK) bad++;
  for (size_t i = threadIdx.x; i < (size_t)ts * cnt; i += blockDim.x)
    if (B[i] != (u64)sh::team_pe(mine, (int)(i / cnt)) * 131 + i % cnt) bad++;
  if (sh::team_sync_block(d, mine) != B200SHMEM_OK) bad++;
  for (size_t i = threadIdx.x; i < (size_t)ts * cnt; i += blockDim.x) A[i] = (u64)me * 100000 + (u64)(i / cnt) * 1000 + i % cnt;
  __syncthreads();
  if (sh::alltoallmem_block(d, mine, B, A, cnt * 8) != B200SHMEM_OK) bad++;
  for (size_t i = threadIdx.x; i < (size_t)ts * cnt; i += blockDim.x)
    if (B[i] != (u64)sh::team_pe(mine, (int)(i / cnt)) * 100000 + (u64)ti * 1000 + i % cnt) bad++;
  for (size_t i = threadIdx.x; i < cnt; i += blockDim.x) R[i] = (u64)me + i;
  __syncthreads();
  if (sh::sum_reduce_block(d, mine, R, R, cnt) != B200SHMEM_OK) bad++;
  u64 peSum = 0;
  for (int m = 0; m < ts; m++) peSum += (u64)sh::team_pe(mine, m);
  for (size_t i = threadIdx.x; i < cnt; i += blockDim.x)
    if (R[i] != (u64)ts * i + peSum) bad++;
  if (sub.idx >= 0) {   // a team of a team: its members only
    for (size_t i = threadIdx.x; i < cnt; i += blockDim.x) A[i] = (u64)((me * 5 + i) % 11);
    __syncthreads();
    if (sh::max_reduce_block(d, sub, B, A, cnt) != B200SHMEM_OK) bad++;
    for (size_t i = threadIdx.x; i < cnt; i += blockDim.x) {
      u64 m = 0;
      for (int k = 0; k < sub.size; k++) m = max(m, (u64)((sh::team_pe(sub, k) * 5 + i) % 11));
      if (B[i] != m) bad++;
    }
  }
  if (sh::barrier_all_block(d) != B200SHMEM_OK) bad++;
  if (bad) atomicAdd(errors, bad);
}
__global__ void kSelftestTeams(b200shmem_dev_t d, b200shmem_team_t mine, b200shmem_team_t sub, unsigned long long* buf, size_t cnt, int* errors) {
  teamsBody(d, mine, sub, buf, cnt, errors);
}
__global__ void kTeamSync(b200shmem_dev_t d, b200shmem_team_t t) { b200shmem::team_sync_block(d, t); }

// Several PEs on one GPU: block r of ONE cooperative launch is PE r (kernels of PEs that wait on one another must never
// be separate launches on one GPU). The bodies are the ones above, each on its PE's own device context.
struct EmuShmemPack {
  b200shmem_dev_t d[B200SHMEM_MAX_PES];
  unsigned long long* data[B200SHMEM_MAX_PES];
  unsigned long long* src[B200SHMEM_MAX_PES];
  unsigned long long* sig[B200SHMEM_MAX_PES];
  unsigned long long* words[B200SHMEM_MAX_PES];
  unsigned long long* coll[B200SHMEM_MAX_PES];
  b200shmem_team_t mine[B200SHMEM_MAX_PES], sub[B200SHMEM_MAX_PES];
  size_t collCount;
  size_t count;
  int rounds, iters;
  int* errors;
};
__global__ void kEmuRing(const EmuShmemPack* p) {
  const int r = blockIdx.x;
  ringBody(p->d[r], p->data[r], p->src[r], p->sig[r], p->count, p->rounds, p->errors);
}
__global__ void kEmuAtomics(const EmuShmemPack* p) {
  const int r = blockIdx.x;
  atomicsBody(p->d[r], p->words[r], p->iters, p->errors);
}
__global__ void kEmuColl(const EmuShmemPack* p) {
  const int r = blockIdx.x;
  collBody(p->d[r], p->coll[r], p->collCount, p->errors);
}
__global__ void kEmuTeams(const EmuShmemPack* p) {
  const int r = blockIdx.x;
  teamsBody(p->d[r], p->mine[r], p->sub[r], p->coll[r], p->collCount, p->errors);
}

struct DevGuard {
  int prev = -1, want;
  explicit DevGuard(int dev) : want(dev) {
    cudaGetDevice(&prev);
    if (prev != want) cudaSetDevice(want);
  }
  ~DevGuard() {
    if (prev != want && prev >= 0) cudaSetDevice(prev);
  }
};

}  // namespace

extern "C" {

ncclResult_t b200shmem_init(ncclComm_t comm, size_t heapBytes, b200shmem_ctx_t* out) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!out || heapBytes == 0) BFAIL(ncclInvalidArgument, "b200shmem_init: bad arguments");
  if (c->nranks > B200SHMEM_MAX_PES) BFAIL(ncclInvalidArgument, "b200shmem_init: at most %d PEs", B200SHMEM_MAX_PES);
  std::unique_ptr<b200shmem_ctx> ctx(new b200shmem_ctx());
  ctx->comm = c;
  void* p = nullptr;
  BCHECK(commSymAlloc(c, heapBytes + kReserved, &p));
  ctx->heap = (char*)p;
  ctx->heapBytes = heapBytes + kReserved;
  DevGuard g(c->cudaDev);
  BCUDA(cudaMalloc(&ctx->devState, kDevStateBytes));
  BCUDA(cudaMemset(ctx->devState, 0, kDevStateBytes));
  b200shmem_dev_t& d = ctx->dev;
  d.pe = c->rank;
  d.npes = c->nranks;
  size_t off = 0;
  Window* w;
  {
    std::lock_guard<std::mutex> lk(c->mu);
    w = c->findWindow(p, 1, &off);
  }
  if (!w) BFAIL(ncclInternalError, "b200shmem_init: heap window not found");
  for (int pe = 0; pe < c->nranks; pe++) d.heap[pe] = w->seg.peer[pe];
  d.heapMc = w->seg.mc;
  d.heapBytes = ctx->heapBytes;
  d.syncFlags = (unsigned long long*)ctx->heap;
  d.syncEpoch = (unsigned long long*)ctx->devState;
  d.status = (int*)((char*)ctx->devState + 16);
  d.timeoutNs = (unsigned long long)Flags::get().waitTimeoutMs * 1000000ull;
  ctx->freeList[kReserved] = heapBytes;
  *out = ctx.release();
  return ncclSuccess;
}

ncclResult_t b200shmem_finalize(b200shmem_ctx_t ctx) {
  if (!ctx) return ncclSuccess;
  DevGuard g(ctx->comm->cudaDev);
  cudaDeviceSynchronize();
  for (int i = 0; i < ctx->dmaReady; i++) {
    cudaStreamDestroy(ctx->dmaStream[i]);
    cudaEventDestroy(ctx->dmaJoin[i]);
  }
  if (ctx->dmaFork) cudaEventDestroy(ctx->dmaFork);
  ncclResult_t r = commSymFree(ctx->comm, ctx->heap);
  if (ctx->devState) cudaFree(ctx->devState);
  delete ctx;
  return r;
}

int b200shmem_my_pe(b200shmem_ctx_t ctx) { return ctx ? ctx->dev.pe : -1; }
int b200shmem_n_pes(b200shmem_ctx_t ctx) { return ctx ? ctx->dev.npes : 0; }

void* b200shmem_align(b200shmem_ctx_t ctx, size_t alignment, size_t size) {
  if (!ctx || size == 0) return nullptr;
  if (alignment < kAlign) alignment = kAlign;
  if (alignment & (alignment - 1)) return nullptr;
  size = (size + kAlign - 1) / kAlign * kAlign;
  std::lock_guard<std::mutex> lk(ctx->mu);
  for (auto it = ctx->freeList.begin(); it != ctx->freeList.end(); ++it) {
    const size_t start = it->first, len = it->second;
    const size_t aligned = (start + alignment - 1) / alignment * alignment;
    if (aligned + size > start + len) continue;
    const size_t tailStart = aligned + size, tailLen = start + len - tailStart;
    ctx->freeList.erase(it);
    if (aligned > start) ctx->freeList[start] = aligned - start;
    if (tailLen) ctx->freeList[tailStart] = tailLen;
    ctx->live[aligned] = size;
    return ctx->heap + aligned;
  }
  return nullptr;
}
void* b200shmem_malloc(b200shmem_ctx_t ctx, size_t size) { return b200shmem_align(ctx, kAlign, size); }

void b200shmem_free(b200shmem_ctx_t ctx, void* ptr) {
  if (!ctx || !ptr) return;
  std::lock_guard<std::mutex> lk(ctx->mu);
  const size_t off = (char*)ptr - ctx->heap;
  auto it = ctx->live.find(off);
  if (it == ctx->live.end()) return;
  size_t start = off, len = it->second;
  ctx->live.erase(it);
  // merge with neighbours
  auto next = ctx->freeList.lower_bound(start);
  if (next != ctx->freeList.end() && next->first == start + len) {
    len += next->second;
    next = ctx->freeList.erase(next);
  }
  if (next != ctx->freeList.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second == start) {
      start = prev->first;
      len += prev->second;
      ctx->freeList.erase(prev);
    }
  }
  ctx->freeList[start] = len;
}

void* b200shmem_ptr(b200shmem_ctx_t ctx, const void* ptr, int pe) {
  if (!ctx || pe < 0 || pe >= ctx->dev.npes) return nullptr;
  const size_t off = (const char*)ptr - ctx->heap;
  if (off >= ctx->heapBytes) return nullptr;
  return ctx->dev.heap[pe] + off;
}
void* b200shmem_mc_ptr(b200shmem_ctx_t ctx, const void* ptr) {
  if (!ctx || !ctx->dev.heapMc) return nullptr;
  const size_t off = (const char*)ptr - ctx->heap;
  if (off >= ctx->heapBytes) return nullptr;
  return ctx->dev.heapMc + off;
}

ncclResult_t b200shmem_device_ctx(b200shmem_ctx_t ctx, b200shmem_dev_t* out) {
  if (!ctx || !out) BFAIL(ncclInvalidArgument, "b200shmem_device_ctx: null argument");
  *out = ctx->dev;
  return ncclSuccess;
}

// ---- teams ---------------------------------------------------------------------------------------------------------------
ncclResult_t b200shmem_team_world(b200shmem_ctx_t ctx, b200shmem_team_t* team) {
  if (!ctx || !team) BFAIL(ncclInvalidArgument, "b200shmem_team_world: null argument");
  *team = b200shmem_team_t{0, 1, ctx->dev.npes, ctx->dev.pe, ctx->dev.syncFlags, ctx->dev.syncEpoch};
  return ncclSuccess;
}

ncclResult_t b200shmem_team_split_strided(b200shmem_ctx_t ctx, const b200shmem_team_t* parent, int start, int stride, int size, b200shmem_team_t* team) {
  if (!ctx || !team) BFAIL(ncclInvalidArgument, "b200shmem_team_split_strided: null argument");
  b200shmem_team_t world;
  BCHECK(b200shmem_team_world(ctx, &world));
  const b200shmem_team_t& par = parent ? *parent : world;
  if (size < 1 || stride < 1 || start < 0 || start + (size - 1) * stride >= par.size)
    BFAIL(ncclInvalidArgument, "b200shmem_team_split_strided: members %d + i * %d, i < %d, do not lie inside a parent of %d", start, stride, size, par.size);
  int slot;
  {
    std::lock_guard<std::mutex> lk(ctx->mu);
    if (ctx->teamSlots >= B200SHMEM_MAX_TEAMS) BFAIL(ncclInvalidUsage, "b200shmem_team_split_strided: at most %d teams per context", B200SHMEM_MAX_TEAMS - 1);
    slot = ctx->teamSlots++;   // every PE makes the same calls in the same order, so the slots agree
  }
  team->start = par.start + start * par.stride;
  team->stride = stride * par.stride;
  team->size = size;
  const int off = ctx->dev.pe - team->start;
  team->idx = (off >= 0 && off % team->stride == 0 && off / team->stride < size) ? off / team->stride : -1;
  team->syncFlags = (unsigned long long*)(ctx->heap + 64 * (size_t)slot);
  team->syncEpoch = (unsigned long long*)((char*)ctx->devState + 64 + 8 * (size_t)slot);
  return ncclSuccess;
}

void b200shmem_team_destroy(b200shmem_ctx_t, b200shmem_team_t* team) {
  if (team) *team = b200shmem_team_t{0, 1, 0, -1, nullptr, nullptr};
}
int b200shmem_team_my_pe(const b200shmem_team_t* team) { return team ? team->idx : -1; }
int b200shmem_team_n_pes(const b200shmem_team_t* team) { return team ? team->size : 0; }
int b200shmem_team_translate_pe(const b200shmem_team_t* src, int idx, const b200shmem_team_t* dst) {
  if (!src || !dst || idx < 0 || idx >= src->size || dst->size < 1) return -1;
  const int off = src->start + idx * src->stride - dst->start;
  if (off < 0 || off % dst->stride) return -1;
  return off / dst->stride < dst->size ? off / dst->stride : -1;
}

ncclResult_t b200shmem_team_sync_on_stream(b200shmem_ctx_t ctx, const b200shmem_team_t* team, cudaStream_t stream) {
  if (!ctx || !team) BFAIL(ncclInvalidArgument, "b200shmem_team_sync_on_stream: null argument");
  if (team->idx < 0) BFAIL(ncclInvalidUsage, "b200shmem_team_sync_on_stream: this PE is not a member of the team");
  DevGuard g(ctx->comm->cudaDev);
  kTeamSync<<<1, 32, 0, stream>>>(ctx->dev, *team);
  BCUDA(cudaGetLastError());
  return ncclSuccess;
}

ncclResult_t b200shmem_putmem_on_stream(b200shmem_ctx_t ctx, void* dest, const void* source, size_t bytes, int pe, cudaStream_t stream) {
  void* r = b200shmem_ptr(ctx, dest, pe);
  if (!r) BFAIL(ncclInvalidArgument, "b200shmem_putmem: destination is not in the symmetric heap");
  DevGuard g(ctx->comm->cudaDev);
  BCUDA(launchCopy(r, source, bytes, 0, stream));
  return ncclSuccess;
}
ncclResult_t b200shmem_getmem_on_stream(b200shmem_ctx_t ctx, void* dest, const void* source, size_t bytes, int pe, cudaStream_t stream) {
  void* r = b200shmem_ptr(ctx, source, pe);
  if (!r) BFAIL(ncclInvalidArgument, "b200shmem_getmem: source is not in the symmetric heap");
  DevGuard g(ctx->comm->cudaDev);
  BCUDA(launchCopy(dest, r, bytes, 0, stream));
  return ncclSuccess;
}
ncclResult_t b200shmem_putmem_signal_on_stream(b200shmem_ctx_t ctx, void* dest, const void* source, size_t bytes, unsigned long long* sigAddr,
                                               unsigned long long signal, int sigOp, int pe, cudaStream_t stream) {
  BCHECK(b200shmem_putmem_on_stream(ctx, dest, source, bytes, pe, stream));
  if (!b200shmem_ptr(ctx, sigAddr, pe)) BFAIL(ncclInvalidArgument, "b200shmem_putmem_signal: signal word is not in the symmetric heap");
  DevGuard g(ctx->comm->cudaDev);
  kSignal<<<1, 32, 0, stream>>>(ctx->dev, sigAddr, signal, sigOp, pe);
  BCUDA(cudaGetLastError());
  return ncclSuccess;
}
ncclResult_t b200shmem_signal_wait_until_on_stream(b200shmem_ctx_t ctx, unsigned long long* sigAddr, int cmp, unsigned long long value, cudaStream_t stream) {
  if (!ctx) BFAIL(ncclInvalidArgument, "null context");
  DevGuard g(ctx->comm->cudaDev);
  kSignalWait<<<1, 32, 0, stream>>>(ctx->dev, sigAddr, cmp, value);
  BCUDA(cudaGetLastError());
  return ncclSuccess;
}
ncclResult_t b200shmem_barrier_all_on_stream(b200shmem_ctx_t ctx, cudaStream_t stream) {
  if (!ctx) BFAIL(ncclInvalidArgument, "null context");
  DevGuard g(ctx->comm->cudaDev);
  kBarrierAll<<<1, 32, 0, stream>>>(ctx->dev);
  BCUDA(cudaGetLastError());
  return ncclSuccess;
}

int b200shmem_take_status(b200shmem_ctx_t ctx) {
  if (!ctx) return -1;
  DevGuard g(ctx->comm->cudaDev);
  int v = 0;
  if (cudaMemcpy(&v, ctx->dev.status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (v) cudaMemset(ctx->dev.status, 0, sizeof(int));
  return v;
}

ncclResult_t b200shmem_selftest_ring(b200shmem_ctx_t ctx, size_t count, int rounds, cudaStream_t stream, int* errors) {
  if (!ctx || !errors) BFAIL(ncclInvalidArgument, "null argument");
  DevGuard g(ctx->comm->cudaDev);
  unsigned long long* data = (unsigned long long*)b200shmem_malloc(ctx, 2 * count * 8);
  unsigned long long* sig = (unsigned long long*)b200shmem_malloc(ctx, 256);
  if (!data || !sig) BFAIL(ncclSystemError, "b200shmem_selftest_ring: symmetric heap too small");
  unsigned long long* src = nullptr;
  int* derr = nullptr;
  BCUDA(cudaMalloc(&src, count * 8));
  BCUDA(cudaMalloc(&derr, sizeof(int)));
  BCUDA(cudaMemsetAsync(derr, 0, sizeof(int), stream));
  BCUDA(cudaMemsetAsync(sig, 0, 256, stream));
  BCHECK(b200shmem_barrier_all_on_stream(ctx, stream));  // signals are zero everywhere before anyone puts
  kSelftestRing<<<1, 256, 0, stream>>>(ctx->dev, data, src, sig, count, rounds, derr);
  BCUDA(cudaGetLastError());
  BCUDA(cudaMemcpyAsync(errors, derr, sizeof(int), cudaMemcpyDeviceToHost, stream));
  BCUDA(cudaStreamSynchronize(stream));
  cudaFree(src);
  cudaFree(derr);
  BCHECK(ctx->comm->boot.barrier());
  b200shmem_free(ctx, sig);
  b200shmem_free(ctx, data);
  return ncclSuccess;
}

ncclResult_t b200shmem_selftest_atomics(b200shmem_ctx_t ctx, int iters, cudaStream_t stream, int* errors) {
  if (!ctx || !errors) BFAIL(ncclInvalidArgument, "null argument");
  DevGuard g(ctx->comm->cudaDev);
  unsigned long long* words = (unsigned long long*)b200shmem_malloc(ctx, 256);
  if (!words) BFAIL(ncclSystemError, "b200shmem_selftest_atomics: symmetric heap too small");
  int* derr = nullptr;
  BCUDA(cudaMalloc(&derr, sizeof(int)));
  BCUDA(cudaMemsetAsync(derr, 0, sizeof(int), stream));
  BCUDA(cudaMemsetAsync(words, 0, 256, stream));
  BCHECK(b200shmem_barrier_all_on_stream(ctx, stream));
  kSelftestAtomics<<<1, 32, 0, stream>>>(ctx->dev, words, iters, derr);
  BCUDA(cudaGetLastError());
  BCUDA(cudaMemcpyAsync(errors, derr, sizeof(int), cudaMemcpyDeviceToHost, stream));
  BCUDA(cudaStreamSynchronize(stream));
  cudaFree(derr);
  BCHECK(ctx->comm->boot.barrier());
  b200shmem_free(ctx, words);
  return ncclSuccess;
}

// Words of the symmetric buffer the collectives self-test needs for `count` elements per block.
static size_t collWords(int npes, size_t count) { return 2 * (size_t)npes * count + count + 8; }

ncclResult_t b200shmem_selftest_collectives(b200shmem_ctx_t ctx, size_t count, cudaStream_t stream, int* errors) {
  if (!ctx || !errors || count < 2) BFAIL(ncclInvalidArgument, "b200shmem_selftest_collectives: bad arguments");
  DevGuard g(ctx->comm->cudaDev);
  const size_t bytes = collWords(ctx->dev.npes, count) * 8;
  unsigned long long* buf = (unsigned long long*)b200shmem_malloc(ctx, bytes);
  if (!buf) BFAIL(ncclSystemError, "b200shmem_selftest_collectives: symmetric heap too small");
  int* derr = nullptr;
  BCUDA(cudaMalloc(&derr, sizeof(int)));
  BCUDA(cudaMemsetAsync(derr, 0, sizeof(int), stream));
  BCUDA(cudaMemsetAsync(buf, 0, bytes, stream));
  BCHECK(b200shmem_barrier_all_on_stream(ctx, stream));  // the flag words are zero everywhere before anyone writes one
  kSelftestColl<<<1, 256, 0, stream>>>(ctx->dev, buf, count, derr);
  BCUDA(cudaGetLastError());
  BCUDA(cudaMemcpyAsync(errors, derr, sizeof(int), cudaMemcpyDeviceToHost, stream));
  BCUDA(cudaStreamSynchronize(stream));
  cudaFree(derr);
  BCHECK(ctx->comm->boot.barrier());
  b200shmem_free(ctx, buf);
  return ncclSuccess;
}

// The PEs split into the even and the odd ones, the even team once more into every second member; the same calls on every PE.
static ncclResult_t makeSelftestTeams(b200shmem_ctx_t ctx, b200shmem_team_t* mine, b200shmem_team_t* sub) {
  const int n = ctx->dev.npes;
  b200shmem_team_t even{}, odd{0, 1, 0, -1, nullptr, nullptr};
  BCHECK(b200shmem_team_split_strided(ctx, nullptr, 0, 2, (n + 1) / 2, &even));
  if (n >= 2) BCHECK(b200shmem_team_split_strided(ctx, nullptr, 1, 2, n / 2, &odd));
  *sub = b200shmem_team_t{0, 1, 0, -1, nullptr, nullptr};
  if (even.size >= 2) BCHECK(b200shmem_team_split_strided(ctx, &even, 0, 2, (even.size + 1) / 2, sub));
  *mine = (ctx->dev.pe & 1) ? odd : even;
  return ncclSuccess;
}

ncclResult_t b200shmem_selftest_teams(b200shmem_ctx_t ctx, size_t count, cudaStream_t stream, int* errors) {
  if (!ctx || !errors || count < 2) BFAIL(ncclInvalidArgument, "b200shmem_selftest_teams: bad arguments");
  DevGuard g(ctx->comm->cudaDev);
  b200shmem_team_t mine, sub;
  BCHECK(makeSelftestTeams(ctx, &mine, &sub));
  const size_t bytes = collWords(ctx->dev.npes, count) * 8;
  unsigned long long* buf = (unsigned long long*)b200shmem_malloc(ctx, bytes);
  if (!buf) BFAIL(ncclSystemError, "b200shmem_selftest_teams: symmetric heap too small");
  int* derr = nullptr;
  BCUDA(cudaMalloc(&derr, sizeof(int)));
  BCUDA(cudaMemsetAsync(derr, 0, sizeof(int), stream));
  BCUDA(cudaMemsetAsync(buf, 0, bytes, stream));
  BCHECK(b200shmem_barrier_all_on_stream(ctx, stream));
  kSelftestTeams<<<1, 256, 0, stream>>>(ctx->dev, mine, sub, buf, count, derr);
  BCUDA(cudaGetLastError());
  BCHECK(b200shmem_team_sync_on_stream(ctx, &mine, stream));   // the stream-ordered form, on the team's own counter
  BCUDA(cudaMemcpyAsync(errors, derr, sizeof(int), cudaMemcpyDeviceToHost, stream));
  BCUDA(cudaStreamSynchronize(stream));
  cudaFree(derr);
  BCHECK(ctx->comm->boot.barrier());
  b200shmem_free(ctx, buf);
  return ncclSuccess;
}

// ---- copy-engine transfers -----------------------------------------------------------------------------------------
// The reference runtime moves bulk peer data with DMA engines and may gang several engines on one copy
// (rocr-runtime core/runtime/amd_gpu_agent.cpp:1013-1108); the count it gangs comes from the link (amd_topology.cpp:442-484).
// Here a transfer is a cudaMemcpyAsync between this PE's mapping of two heaps, which the driver runs on a copy engine,
// and a large one is cut into page-aligned parts on side streams that fork from and join the caller's stream with
// events, so it stays stream-ordered (and capturable) as a whole. No SM takes part: the path for bulk data that must
// not compete with running GEMMs (pipeline stages, checkpoint traffic).

int b200shmem_dma_plan(size_t bytes, int gang, size_t* offsets, size_t* lengths) {
  if (gang <= 0) {
    const long env = Flags::get().dmaGang;
    gang = env > 0 ? (int)env : (bytes >= (64u << 20) ? 4 : bytes >= (8u << 20) ? 2 : 1);
  }
  if (gang > B200SHMEM_MAX_DMA_GANG) gang = B200SHMEM_MAX_DMA_GANG;
  constexpr size_t kPart = 64u << 10;  // parts are multiples of 64 KiB, so that none is too small to be worth an engine
  const size_t units = (bytes + kPart - 1) / kPart;
  if ((size_t)gang > units) gang = units ? (int)units : 1;
  size_t off = 0;
  for (int i = 0; i < gang; i++) {
    const size_t u = units / gang + ((size_t)i < units % gang ? 1 : 0);
    size_t len = u * kPart;
    if (off + len > bytes) len = bytes - off;
    if (offsets) offsets[i] = off;
    if (lengths) lengths[i] = len;
    off += len;
  }
  return gang;
}

static ncclResult_t dmaSetup(b200shmem_ctx_t ctx, int gang) {
  std::lock_guard<std::mutex> lk(ctx->mu);
  if (!ctx->dmaFork) BCUDA(cudaEventCreateWithFlags(&ctx->dmaFork, cudaEventDisableTiming));
  while (ctx->dmaReady < gang) {
    const int i = ctx->dmaReady;
    BCUDA(cudaStreamCreateWithFlags(&ctx->dmaStream[i], cudaStreamNonBlocking));
    BCUDA(cudaEventCreateWithFlags(&ctx->dmaJoin[i], cudaEventDisableTiming));
    ctx->dmaReady = i + 1;
  }
  return ncclSuccess;
}

static ncclResult_t dmaCopy(b200shmem_ctx_t ctx, char* dst, const char* src, size_t bytes, int gang, cudaStream_t stream) {
  if (bytes == 0) return ncclSuccess;
  size_t off[B200SHMEM_MAX_DMA_GANG], len[B200SHMEM_MAX_DMA_GANG];
  const int g = b200shmem_dma_plan(bytes, gang, off, len);
  DevGuard dg(ctx->comm->cudaDev);
  if (g == 1) {
    BCUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream));
    return ncclSuccess;
  }
  BCHECK(dmaSetup(ctx, g - 1));
  // The fork / join events are shared by all transfers of the context: one transfer is enqueued at a time.
  static std::mutex enqueueMu;
  std::lock_guard<std::mutex> lk(enqueueMu);
  // Part 0 stays on the caller's stream; the others fork after everything already queued there and join before
  // anything queued later.
  BCUDA(cudaEventRecord(ctx->dmaFork, stream));
  for (int i = 1; i < g; i++) {
    cudaStream_t s = ctx->dmaStream[i - 1];
    BCUDA(cudaStreamWaitEvent(s, ctx->dmaFork, 0));
    BCUDA(cudaMemcpyAsync(dst + off[i], src + off[i], len[i], cudaMemcpyDeviceToDevice, s));
    BCUDA(cudaEventRecord(ctx->dmaJoin[i - 1], s));
  }
  BCUDA(cudaMemcpyAsync(dst + off[0], src + off[0], len[0], cudaMemcpyDeviceToDevice, stream));
  for (int i = 1; i < g; i++) BCUDA(cudaStreamWaitEvent(stream, ctx->dmaJoin[i - 1], 0));
  return ncclSuccess;
}

ncclResult_t b200shmem_putmem_dma_on_stream(b200shmem_ctx_t ctx, void* dest, const void* source, size_t bytes, int pe, int gang, cudaStream_t stream) {
  void* r = b200shmem_ptr(ctx, dest, pe);
  if (!r) BFAIL(ncclInvalidArgument, "b200shmem_putmem_dma: destination is not in the symmetric heap");
  return dmaCopy(ctx, (char*)r, (const char*)source, bytes, gang, stream);
}
ncclResult_t b200shmem_getmem_dma_on_stream(b200shmem_ctx_t ctx, void* dest, const void* source, size_t bytes, int pe, int gang, cudaStream_t stream) {
  void* r = b200shmem_ptr(ctx, source, pe);
  if (!r) BFAIL(ncclInvalidArgument, "b200shmem_getmem_dma: source is not in the symmetric heap");
  return dmaCopy(ctx, (char*)dest, (const char*)r, bytes, gang, stream);
}
ncclResult_t b200shmem_putmem_signal_dma_on_stream(b200shmem_ctx_t ctx, void* dest, const void* source, size_t bytes, unsigned long long* sigAddr,
                                                   unsigned long long signal, int sigOp, int pe, int gang, cudaStream_t stream) {
  if (!b200shmem_ptr(ctx, sigAddr, pe)) BFAIL(ncclInvalidArgument, "b200shmem_putmem_signal_dma: signal word is not in the symmetric heap");
  BCHECK(b200shmem_putmem_dma_on_stream(ctx, dest, source, bytes, pe, gang, stream));
  // The signal follows the joined copies in stream order; one warp stores it with release semantics at system scope.
  DevGuard g(ctx->comm->cudaDev);
  kSignal<<<1, 32, 0, stream>>>(ctx->dev, sigAddr, signal, sigOp, pe);
  BCUDA(cudaGetLastError());
  return ncclSuccess;
}
int b200shmem_dma_engines(b200shmem_ctx_t ctx) {
  if (!ctx) return -1;
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrAsyncEngineCount, ctx->comm->cudaDev) != cudaSuccess) return -1;
  return v;
}

// Device-initiated communication between `n` PEs that share the current GPU (communicators created under
// B200COLL_EMULATE_RANKS=1): the put+signal ring and the remote-atomics check of the self-tests above, every PE a block of
// one cooperative kernel. *errors = mismatches plus waits that ran out.
ncclResult_t b200shmem_emu_selftest(ncclComm_t* comms, int n, size_t count, int rounds, int iters, int* errors) {
  if (!comms || !errors || n < 2 || n > B200SHMEM_MAX_PES || count == 0) BFAIL(ncclInvalidArgument, "b200shmem_emu_selftest: bad arguments");
  *errors = 0;
  std::vector<b200shmem_ctx_t> ctx(n, nullptr);
  std::vector<ncclResult_t> rs(n, ncclSuccess);
  const size_t collCount = 96;
  const size_t heap = 2 * count * 8 + collWords(n, collCount) * 8 + (4u << 20);
  auto onEveryPe = [&](auto fn) {  // the heap calls are collective over the communicator: one thread per PE
    std::vector<std::thread> th;
    for (int r = 0; r < n; r++)
      th.emplace_back([&, r] {
        tlsEmuCall = true;
        rs[r] = fn(r);
        tlsEmuCall = false;
      });
    for (auto& t : th) t.join();
    for (ncclResult_t r : rs)
      if (r != ncclSuccess) return r;
    return ncclSuccess;
  };
  BCHECK(onEveryPe([&](int r) { return b200shmem_init(comms[r], heap, &ctx[r]); }));
  EmuShmemPack pack{};
  pack.count = count;
  pack.rounds = rounds;
  pack.iters = iters;
  pack.collCount = collCount;
  int* derr = nullptr;
  BCUDA(cudaMalloc(&derr, sizeof(int)));
  BCUDA(cudaMemset(derr, 0, sizeof(int)));
  pack.errors = derr;
  for (int r = 0; r < n; r++) {
    pack.d[r] = ctx[r]->dev;
    pack.data[r] = (unsigned long long*)b200shmem_malloc(ctx[r], 2 * count * 8);
    pack.sig[r] = (unsigned long long*)b200shmem_malloc(ctx[r], 256);
    pack.words[r] = (unsigned long long*)b200shmem_malloc(ctx[r], 256);
    pack.coll[r] = (unsigned long long*)b200shmem_malloc(ctx[r], collWords(n, collCount) * 8);
    if (pack.coll[r]) BCUDA(cudaMemset(pack.coll[r], 0, collWords(n, collCount) * 8));
    if (!pack.data[r] || !pack.sig[r] || !pack.words[r] || !pack.coll[r]) BFAIL(ncclSystemError, "b200shmem_emu_selftest: symmetric heap too small");
    BCUDA(cudaMalloc(&pack.src[r], count * 8));
    BCUDA(cudaMemset(pack.sig[r], 0, 256));
    BCUDA(cudaMemset(pack.words[r], 0, 256));
  }
  for (int r = 0; r < n; r++) BCHECK(makeSelftestTeams(ctx[r], &pack.mine[r], &pack.sub[r]));
  EmuShmemPack* dpack = nullptr;
  BCUDA(cudaMalloc(&dpack, sizeof(pack)));
  BCUDA(cudaMemcpy(dpack, &pack, sizeof(pack), cudaMemcpyHostToDevice));
  BCUDA(cudaDeviceSynchronize());
  void* args[] = {(void*)&dpack};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)kEmuRing, dim3(n), dim3(256), args, 0, 0);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaLaunchCooperativeKernel((const void*)kEmuAtomics, dim3(n), dim3(32), args, 0, 0);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaLaunchCooperativeKernel((const void*)kEmuColl, dim3(n), dim3(256), args, 0, 0);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaLaunchCooperativeKernel((const void*)kEmuTeams, dim3(n), dim3(256), args, 0, 0);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "b200shmem_emu_selftest: %s", cudaGetErrorString(e));
  BCUDA(cudaMemcpy(errors, derr, sizeof(int), cudaMemcpyDeviceToHost));
  for (int r = 0; r < n; r++) {
    int st = 0;
    if (cudaMemcpy(&st, ctx[r]->dev.status, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess && st) (*errors)++;
    cudaFree(pack.src[r]);
  }
  cudaFree(derr);
  cudaFree(dpack);
  BCHECK(onEveryPe([&](int r) { return b200shmem_finalize(ctx[r]); }));
  return ncclSuccess;
}

}  // extern "C"
