// Several ranks of one communicator on ONE GPU, played by ONE cooperative kernel.
//
// Ranks that wait on one another must never run as separate launches on one GPU: nothing makes them run together.
// Here block (r * lanes + b) of a single cooperative grid runs lane b of rank r, executing the very same kernel bodies
// the library launches per rank (kernels.cuh is compiled a second time with its __global__ functions turned into
// device functions and blockIdx / gridDim turned into the emulated rank's view), on the ranks' real communicators:
// workspaces, barrier slots, staging halves, sequence numbers and plans are those of commCreate / the planner. The
// cooperative launch guarantees that all blocks are resident, so the inter-rank waits complete; they stay bounded as
// always. Peer loads and stores become local loads and stores, the in-switch path is absent (one device cannot form a
// multicast group), everything else — pipelining, chunk geometry, bulk asynchronous loads, flag-in-data lines — runs
// as on eight GPUs. For tests on a single GPU; communicators of this kind refuse every other entry point.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <type_traits>
#include <thread>
#include <vector>

#include "../core/comm.h"
#include "../trace/tracer.h"
#include "b200coll/api_trace.h"
#include "b200coll/fused.h"
#include "b200coll/nccl.h"
#include "b200coll/shmem.h"
#include "device.h"
#include "enqueue.h"
#include "launch.h"

namespace b200 {
namespace emu {
struct Dim { unsigned x, y, z; };
__device__ unsigned gLanes;  // lanes (CTAs) per emulated rank of the running launch
__device__ __forceinline__ Dim block() {
  unsigned r;
  asm volatile("mov.u32 %0, %%ctaid.x;" : "=r"(r));
  return Dim{r % gLanes, 0, 0};
}
__device__ __forceinline__ Dim grid() { return Dim{gLanes, 1, 1}; }
}  // namespace emu
}  // namespace b200

// ---- the library's kernels once more, as device functions seeing the emulated rank's grid -------------------------
// prims.cuh comes in here, under the same substitution: the inter-rank barrier picks its slots by the lane index.
#pragma push_macro("__global__")
#pragma push_macro("__launch_bounds__")
#pragma push_macro("__grid_constant__")
#undef __global__
#undef __launch_bounds__
#undef __grid_constant__
#define __global__ __device__ __noinline__
#define __launch_bounds__(...)
#define __grid_constant__
#define blockIdx (::b200::emu::block())
#define gridDim (::b200::emu::grid())
#define B200_MISC_KERNELS 1       // the send/recv kernel too, under names of its own (launch.cu defines the originals)
#define kP2p emuP2p
#define kBarrier emuBarrier
#define kAllToAllDirect emuAllToAllDirect
#define kLLAllGather emuLLAllGather
#include "kernels.cuh"
#undef kLLAllGather
#undef kP2p
#undef kBarrier
#undef kAllToAllDirect
#undef B200_MISC_KERNELS
#define B200_EMU_KERNELS_ONLY 1
// Non-template functions get names of their own here: the library's other object file defines the originals.
#define kReduceScatterCast emuReduceScatterCast
#define kReduceScatterCastDirect emuReduceScatterCastDirect
#define kCastScaleSolo emuCastScaleSolo
#include "../fused/fsdp_kernels.cu"  // the kernels and their helpers only
#undef kReduceScatterCast
#undef kReduceScatterCastDirect
#undef kCastScaleSolo
#undef B200_EMU_KERNELS_ONLY
#undef blockIdx
#undef gridDim
#pragma pop_macro("__grid_constant__")
#pragma pop_macro("__launch_bounds__")
#pragma pop_macro("__global__")

namespace b200 {
namespace emu {

struct Pack {
  DevComm c[kMaxRanks];
  CollArgs a[kMaxRanks];
  LLArgs ll[kMaxRanks];
  int lanes;
  int elemSize;
};

template <typename T, typename Op> __global__ void __launch_bounds__(kReduceThreads) kReduce(const Pack* p) {
  const unsigned r = blockIdx.x / (unsigned)p->lanes;
  kStagedReduce<T, Op, false>(p->c[r], p->a[r]);
}
template <typename T, typename Op> __global__ void __launch_bounds__(kCollThreads) kLL(const Pack* p) {
  const unsigned r = blockIdx.x / (unsigned)p->lanes;
  kLLAllReduce<T, Op>(p->c[r], p->ll[r]);
}
__global__ void __launch_bounds__(kCollThreads) kCopy(const Pack* p) {
  const unsigned r = blockIdx.x / (unsigned)p->lanes;
  kStagedCopy<false>(p->c[r], p->a[r], p->elemSize);
}
__global__ void __launch_bounds__(kCollThreads) kGatherLL(const Pack* p) {
  const unsigned r = blockIdx.x / (unsigned)p->lanes;
  emuLLAllGather(p->c[r], p->ll[r]);
}

struct P2pPack {
  DevComm c[kMaxRanks];
  P2pArgs a[kMaxRanks];
  int lanes;
};
__global__ void __launch_bounds__(kCollThreads) kSendRecv(const P2pPack* p) {
  const unsigned r = blockIdx.x / (unsigned)p->lanes;
  emuP2p(p->c[r], p->a[r]);
}

struct RsCastPack {
  DevComm c[kMaxRanks];
  RsCastArgs a[kMaxRanks];
  int lanes;
};
__global__ void __launch_bounds__(kReduceThreads) kRsCast(const RsCastPack* p) {
  const unsigned r = blockIdx.x / (unsigned)p->lanes;
  emuReduceScatterCast(p->c[r], p->a[r]);
}

static cudaError_t launchCoop(const void* fn, int blocks, int threads, size_t smem, const void* devPack, unsigned lanes, cudaStream_t s) {
  cudaError_t e = cudaMemcpyToSymbolAsync(gLanes, &lanes, sizeof(lanes), 0, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return e;
  if (smem > (48u << 10)) {
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  // Every block must be resident at once; refuse instead of letting waits run into their time limit.
  int perSm = 0, dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, fn, threads, smem);
  if (e != cudaSuccess) return e;
  if (blocks > perSm * sms) return cudaErrorCooperativeLaunchTooLarge;
  void* args[] = {(void*)&devPack};
  return cudaLaunchCooperativeKernel(fn, dim3(blocks), dim3(threads), args, smem, s);
}

template <typename T> static const void* reduceFn(int op, bool ll) {
  switch (op) {
    case ncclSum: return ll ? (const void*)kLL<T, OpSum> : (const void*)kReduce<T, OpSum>;
    case ncclMax: return ll ? (const void*)kLL<T, OpMax> : (const void*)kReduce<T, OpMax>;
    default: return nullptr;
  }
}

}  // namespace emu
}  // namespace b200

using namespace b200;

extern "C" {

// One collective on `n` communicators that share the current GPU (created under B200COLL_EMULATE_RANKS=1), all ranks
// played by one cooperative kernel on `stream`. send[r] / recv[r] are rank r's buffers. Types: float, bfloat16, int32;
// operators of reducing collectives: sum, max, avg. ctasPerRank: 0 = 4.
ncclResult_t b200collEmuCollective(ncclComm_t* comms, int n, int kind, const void* const* send, void* const* recv, size_t count, ncclDataType_t dt,
                                   ncclRedOp_t op, int root, int ctasPerRank, cudaStream_t stream) {
  if (!comms || n < 2 || n > kMaxRanks || !send || !recv) BFAIL(ncclInvalidArgument, "b200collEmuCollective: bad arguments");
  if (dt != ncclFloat32 && dt != ncclBfloat16 && dt != ncclInt32) BFAIL(ncclInvalidArgument, "b200collEmuCollective: float, bfloat16 or int32");
  const bool reducing = kind == COLL_ALLREDUCE || kind == COLL_REDUCESCATTER || kind == COLL_REDUCE;
  if (reducing && op != ncclSum && op != ncclMax && op != ncclAvg) BFAIL(ncclInvalidArgument, "b200collEmuCollective: sum, max or avg");
  struct Scope {
    Scope() { tlsEmuCall = true; }
    ~Scope() { tlsEmuCall = false; }
  } scope;
  emu::Pack pack{};
  Plan first{};
  for (int r = 0; r < n; r++) {
    Comm* c = asComm(comms[r]);
    BCHECK(commCheck(c));
    if (!c->emulated || c->nranks != n || c->rank != r) BFAIL(ncclInvalidUsage, "b200collEmuCollective: comms[%d] must be rank %d of %d ranks sharing one GPU", r, r, n);
    CollReq q{};
    q.kind = kind;
    q.send = send[r];
    q.recv = recv[r];
    q.count = count;
    q.dt = dt;
    q.op = (int)op;
    q.root = root;
    q.comm = c;
    q.stream = stream;
    q.forceCtas = ctasPerRank > 0 ? ctasPerRank : 4;
    Plan plan{};
    if (kind == COLL_ALLTOALL) {  // the staged form for large chunks; `count` elements per pair
      int ctas = 0;
      stagedAllToAllArgs(c, send[r], recv[r], count, dt, q.forceCtas, &pack.a[r], &pack.c[r], &ctas);
      plan.algo = ALGO_P2P;
      plan.ctas = ctas;
      if (r == 0) first = plan;
      continue;
    }
    BCHECK(emuPrepare(q, &plan, &pack.a[r], &pack.ll[r], &pack.c[r]));
    if (r == 0) first = plan;
    if (plan.algo != first.algo || plan.ctas != first.ctas || plan.chunks != first.chunks || plan.direct != first.direct)
      BFAIL(ncclInternalError, "b200collEmuCollective: the ranks planned differently");
  }
  if (first.algo == ALGO_NVLS) BFAIL(ncclInternalError, "b200collEmuCollective: the in-switch path cannot be emulated");
  const bool ll = first.algo == ALGO_LL;
  // Grid per rank and block size exactly as enqueueColl launches them.
  const int lanes = ll ? first.ctas : (reducing ? std::min(2 * first.ctas, kMaxCtas) : first.ctas);
  const int threads = (reducing && !ll) ? kReduceThreads : kCollThreads;
  const size_t smem = (reducing && !ll) ? kBulkSmemBytes : 0;
  pack.lanes = lanes;
  pack.elemSize = (int)dtypeSize(dt);
  emu::Pack* devPack = nullptr;
  BCUDA(cudaMallocAsync((void**)&devPack, sizeof(emu::Pack), stream));
  BCUDA(cudaMemcpyAsync(devPack, &pack, sizeof(pack), cudaMemcpyHostToDevice, stream));
  BCUDA(cudaStreamSynchronize(stream));  // `pack` is a stack object
  const void* fn = nullptr;
  if (reducing) {
    const int base = op == ncclAvg ? (int)ncclSum : (int)op;
    fn = dt == ncclFloat32 ? emu::reduceFn<float>(base, ll) : dt == ncclBfloat16 ? emu::reduceFn<__nv_bfloat16>(base, ll) : emu::reduceFn<int32_t>(base, ll);
  } else {
    fn = ll ? (const void*)emu::kGatherLL : (const void*)emu::kCopy;
  }
  if (!fn) BFAIL(ncclInternalError, "b200collEmuCollective: no kernel for this operator");
  cudaError_t e = emu::launchCoop(fn, n * lanes, threads, smem, devPack, (unsigned)lanes, stream);
  cudaFreeAsync(devPack, stream);
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "b200collEmuCollective: launch of %d x %d blocks failed: %s", n, lanes, cudaGetErrorString(e));
  return ncclSuccess;
}

// All-to-all of `bytesPerPeer` bytes between every pair of emulated ranks, as the grouped send/recv kernel runs it: one
// send and one receive work item per peer and rank, each on the communicator's sub-channels, through the FIFO slots and
// credits of the real workspaces. Rank r's own block is a local copy.
ncclResult_t b200collEmuAllToAll(ncclComm_t* comms, int n, const void* const* send, void* const* recv, size_t bytesPerPeer, cudaStream_t stream) {
  if (!comms || n < 2 || n > kMaxRanks || !send || !recv || bytesPerPeer == 0) BFAIL(ncclInvalidArgument, "b200collEmuAllToAll: bad arguments");
  struct Scope {
    Scope() { tlsEmuCall = true; }
    ~Scope() { tlsEmuCall = false; }
  } scope;
  emu::P2pPack pack{};
  int subs = 0;
  for (int r = 0; r < n; r++) {
    Comm* c = asComm(comms[r]);
    BCHECK(commCheck(c));
    if (!c->emulated || c->nranks != n || c->rank != r) BFAIL(ncclInvalidUsage, "b200collEmuAllToAll: comms[%d] must be rank %d of %d ranks sharing one GPU", r, r, n);
    P2pArgs& pa = pack.a[r];
    for (int d = 1; d < n; d++) {
      const int to = (r + d) % n, from = (r - d + n) % n;
      P2pWork& ws = pa.work[pa.nwork++];
      ws.peer = to;
      ws.isSend = 1;
      ws.src = (const char*)send[r] + (size_t)to * bytesPerPeer;
      ws.dst = nullptr;
      ws.bytes = bytesPerPeer;
      P2pWork& wr = pa.work[pa.nwork++];
      wr.peer = from;
      wr.isSend = 0;
      wr.src = nullptr;
      wr.dst = (char*)recv[r] + (size_t)from * bytesPerPeer;
      wr.bytes = bytesPerPeer;
    }
    BCUDA(cudaMemcpyAsync((char*)recv[r] + (size_t)r * bytesPerPeer, (const char*)send[r] + (size_t)r * bytesPerPeer, bytesPerPeer, cudaMemcpyDeviceToDevice, stream));
    pack.c[r] = c->dev;
    pack.c[r].opSeq = ++c->opSeq;
    pack.c[r].stamp = nullptr;
    subs = c->dev.p2pSubs;
  }
  // All blocks must be resident together: use as many of the communicator's sub-channels as fit. Sender and receiver
  // of a launch agree on the number (it is part of the device view both get), and the FIFOs are empty between launches.
  int perSm = 0, dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  BCUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, (const void*)emu::kSendRecv, kCollThreads, 0));
  const int fit = (perSm * sms) / (n * pack.a[0].nwork);
  if (fit < 1) BFAIL(ncclInternalError, "b200collEmuAllToAll: %d ranks do not fit this GPU", n);
  subs = std::min(subs, fit);
  for (int r = 0; r < n; r++) pack.c[r].p2pSubs = subs;
  const int lanes = pack.a[0].nwork * subs;
  pack.lanes = lanes;
  emu::P2pPack* devPack = nullptr;
  BCUDA(cudaMallocAsync((void**)&devPack, sizeof(pack), stream));
  BCUDA(cudaMemcpyAsync(devPack, &pack, sizeof(pack), cudaMemcpyHostToDevice, stream));
  BCUDA(cudaStreamSynchronize(stream));
  cudaError_t e = emu::launchCoop((const void*)emu::kSendRecv, n * lanes, kCollThreads, 0, devPack, (unsigned)lanes, stream);
  cudaFreeAsync(devPack, stream);
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "b200collEmuAllToAll: launch of %d x %d blocks failed: %s", n, lanes, cudaGetErrorString(e));
  return ncclSuccess;
}

// The fused FSDP gradient reduce-scatter (bf16 in, fp32 out, scaled) on emulated ranks: send[r] holds n * recvcount
// bf16 elements, recv[r] receives rank r's recvcount fp32 sums, through the staged path of b200collReduceScatterCast
// (same chunking and staging parity: rsCastStagedArgs).
ncclResult_t b200collEmuReduceScatterCast(ncclComm_t* comms, int n, const void* const* send, float* const* recv, size_t recvcount, float scale,
                                          int ctasPerRank, cudaStream_t stream) {
  if (!comms || n < 2 || n > kMaxRanks || !send || !recv || recvcount == 0) BFAIL(ncclInvalidArgument, "b200collEmuReduceScatterCast: bad arguments");
  struct Scope {
    Scope() { tlsEmuCall = true; }
    ~Scope() { tlsEmuCall = false; }
  } scope;
  emu::RsCastPack pack{};
  const int lanes = ctasPerRank > 0 ? std::min(ctasPerRank, 16) : 8;
  for (int r = 0; r < n; r++) {
    Comm* c = asComm(comms[r]);
    BCHECK(commCheck(c));
    if (!c->emulated || c->nranks != n || c->rank != r) BFAIL(ncclInvalidUsage, "b200collEmuReduceScatterCast: comms[%d] must be rank %d of %d ranks sharing one GPU", r, r, n);
    pack.a[r] = rsCastStagedArgs(c, send[r], recv[r], recvcount, scale);
    pack.c[r] = c->dev;
    pack.c[r].opSeq = ++c->opSeq;
    pack.c[r].stamp = nullptr;
  }
  pack.lanes = lanes;
  emu::RsCastPack* devPack = nullptr;
  BCUDA(cudaMallocAsync((void**)&devPack, sizeof(pack), stream));
  BCUDA(cudaMemcpyAsync(devPack, &pack, sizeof(pack), cudaMemcpyHostToDevice, stream));
  BCUDA(cudaStreamSynchronize(stream));
  cudaError_t e = emu::launchCoop((const void*)emu::kRsCast, n * lanes, kReduceThreads, 0, devPack, (unsigned)lanes, stream);
  cudaFreeAsync(devPack, stream);
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "b200collEmuReduceScatterCast: launch of %d x %d blocks failed: %s", n, lanes, cudaGetErrorString(e));
  return ncclSuccess;
}

// Self-check on the current GPU: `nranks` emulated ranks, all-reduce (sum, max, avg), reduce-scatter, reduce,
// all-gather and broadcast of `count` elements in float, bfloat16 and int32, out of place, verified on the host against
// sums of small integers (exact in every type). Returns the number of wrong elements, and in *status the first
// asynchronous error of any rank (a bounded wait that ran out shows here). The caller sets B200COLL_EMULATE_RANKS=1 and
// B200COLL_NVLS_ENABLE=0 before the first call of the library in the process.
ncclResult_t b200collEmuSelftest(int nranks, size_t count, long long* wrong, int* status) {
  if (!wrong || !status || nranks < 2 || nranks > kMaxRanks || count == 0) BFAIL(ncclInvalidArgument, "b200collEmuSelftest: bad arguments");
  *wrong = 0;
  *status = 0;
  int dev = 0;
  BCUDA(cudaGetDevice(&dev));
  std::vector<ncclComm_t> comms(nranks);
  std::vector<int> devs(nranks, dev);
  BCHECK(ncclCommInitAll(comms.data(), nranks, devs.data()));
  cudaStream_t st;
  BCUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  const size_t maxElems = count * nranks;
  std::vector<void*> send(nranks), recv(nranks);
  for (int r = 0; r < nranks; r++) {
    BCUDA(cudaMalloc(&send[r], maxElems * 4 + 64));
    BCUDA(cudaMalloc(&recv[r], maxElems * 4 + 64));
  }
  auto value = [](int rank, size_t i, int salt) -> int { return (int)((i * 7 + (size_t)rank * 13 + (size_t)salt * 5) % 9) - 4; };
  const ncclDataType_t types[3] = {ncclFloat32, ncclBfloat16, ncclInt32};
  ncclResult_t res = ncclSuccess;
  int salt = 0;
  for (int ti = 0; ti < 3 && res == ncclSuccess; ti++) {
    const ncclDataType_t dt = types[ti];
    const size_t es = dtypeSize(dt);
    auto encode = [&](std::vector<char>& buf, size_t i, int v) {
      if (dt == ncclFloat32) { float f = (float)v; memcpy(&buf[i * 4], &f, 4); }
      else if (dt == ncclInt32) { int32_t x = v; memcpy(&buf[i * 4], &x, 4); }
      else { __nv_bfloat16 h = __float2bfloat16((float)v); memcpy(&buf[i * 2], &h, 2); }
    };
    auto decode = [&](const std::vector<char>& buf, size_t i) -> double {
      if (dt == ncclFloat32) { float f; memcpy(&f, &buf[i * 4], 4); return f; }
      if (dt == ncclInt32) { int32_t x; memcpy(&x, &buf[i * 4], 4); return x; }
      __nv_bfloat16 h; memcpy(&h, &buf[i * 2], 2); return (double)__bfloat162float(h);
    };
    struct Case { int kind; ncclRedOp_t op; int root; };
    const Case cases[] = {{COLL_ALLREDUCE, ncclSum, 0}, {COLL_ALLREDUCE, ncclMax, 0}, {COLL_ALLREDUCE, ncclAvg, 0}, {COLL_REDUCESCATTER, ncclSum, 0},
                          {COLL_REDUCE, ncclSum, nranks - 1}, {COLL_ALLGATHER, ncclSum, 0}, {COLL_BROADCAST, ncclSum, 1}};
    for (const Case& cs : cases) {
      if (dt == ncclInt32 && cs.op == ncclAvg) continue;  // integer division truncates: covered by the multi-GPU sweep
      salt++;
      const size_t sendElems = cs.kind == COLL_REDUCESCATTER ? count * nranks : count;
      const size_t recvElems = cs.kind == COLL_ALLGATHER ? count * nranks : count;
      std::vector<std::vector<char>> in(nranks, std::vector<char>(sendElems * es));
      for (int r = 0; r < nranks; r++) {
        for (size_t i = 0; i < sendElems; i++) encode(in[r], i, value(r, i, salt));
        BCUDA(cudaMemcpyAsync(send[r], in[r].data(), sendElems * es, cudaMemcpyHostToDevice, st));
        BCUDA(cudaMemsetAsync(recv[r], 0xEE, recvElems * es + 64, st));
      }
      res = b200collEmuCollective(comms.data(), nranks, cs.kind, send.data(), recv.data(), count, dt, cs.op, cs.root, 0, st);
      if (res != ncclSuccess) break;
      BCUDA(cudaStreamSynchronize(st));
      const long long wrongBefore = *wrong;
      long long firstBad = -1, lastBad = -1;
      int firstBadRank = -1;
      for (int r = 0; r < nranks; r++) {
        if (cs.kind == COLL_REDUCE && r != cs.root) continue;
        std::vector<char> out(recvElems * es + 64);
        BCUDA(cudaMemcpy(out.data(), recv[r], out.size(), cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < recvElems; i++) {
          double want = 0;
          if (cs.kind == COLL_ALLGATHER) {
            want = value((int)(i / count), i % count, salt);
          } else if (cs.kind == COLL_BROADCAST) {
            want = value(cs.root, i, salt);
          } else {
            const size_t src = cs.kind == COLL_REDUCESCATTER ? (size_t)r * count + i : i;
            if (cs.op == ncclMax) {
              want = -1e9;
              for (int p = 0; p < nranks; p++) want = std::max(want, (double)value(p, src, salt));
            } else {
              for (int p = 0; p < nranks; p++) want += value(p, src, salt);
              if (cs.op == ncclAvg) want /= nranks;
            }
          }
          const double got = decode(out, i);
          const double tol = cs.op == ncclAvg ? (dt == ncclBfloat16 ? 0.05 : 1e-5) : 0.0;
          if (!(got >= want - tol && got <= want + tol)) {
            (*wrong)++;
            if (firstBad < 0) { firstBad = (long long)i; firstBadRank = r; }
            lastBad = (long long)i;
          }
        }
        for (size_t b = recvElems * es; b < recvElems * es + 64; b++)  // the bytes behind the output keep their fill
          if ((unsigned char)out[b] != 0xEE) (*wrong)++;
      }
      if (*wrong != wrongBefore)
        BWARN("emulated ranks: %lld wrong values in kind %d op %d type %s, %d ranks, count %zu; first at rank %d element %lld, last at element %lld",
              *wrong - wrongBefore, cs.kind, (int)cs.op, dtypeName(dt), nranks, count, firstBadRank, firstBad, lastBad);
    }
  }
  // The fused FSDP gradient path: bf16 gradients of every rank -> this rank's fp32 mean.
  if (res == ncclSuccess) {
    salt++;
    const float scale = 1.0f / (float)nranks;
    std::vector<float*> out32(nranks);
    for (int r = 0; r < nranks; r++) {
      std::vector<__nv_bfloat16> in(count * nranks);
      for (size_t i = 0; i < in.size(); i++) in[i] = __float2bfloat16((float)value(r, i, salt));
      BCUDA(cudaMemcpyAsync(send[r], in.data(), in.size() * 2, cudaMemcpyHostToDevice, st));
      BCUDA(cudaMemsetAsync(recv[r], 0xEE, count * 4 + 64, st));
      BCUDA(cudaStreamSynchronize(st));  // `in` goes out of scope
      out32[r] = (float*)recv[r];
    }
    res = b200collEmuReduceScatterCast(comms.data(), nranks, send.data(), out32.data(), count, scale, 0, st);
    if (res == ncclSuccess) {
      BCUDA(cudaStreamSynchronize(st));
      for (int r = 0; r < nranks; r++) {
        std::vector<char> out(count * 4 + 64);
        BCUDA(cudaMemcpy(out.data(), recv[r], out.size(), cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < count; i++) {
          float sum = 0;
          for (int p = 0; p < nranks; p++) sum += (float)value(p, (size_t)r * count + i, salt);
          float got;
          memcpy(&got, &out[i * 4], 4);
          const float want = sum * scale;
          if (!(got >= want - 1e-6f && got <= want + 1e-6f)) (*wrong)++;
        }
        for (size_t b = count * 4; b < count * 4 + 64; b++)
          if ((unsigned char)out[b] != 0xEE) (*wrong)++;
      }
    }
  }
  // All-to-all through the send/recv FIFOs: rank s sends the block (s, d) to rank d.
  if (res == ncclSuccess) {
    salt++;
    const size_t per = std::min<size_t>(count, (size_t)1 << 20) * 4;  // bytes per pair, several FIFO slots for the larger counts
    const size_t words = per / 4;
    for (int r = 0; r < nranks; r++) {
      std::vector<int32_t> in(words * nranks);
      for (size_t i = 0; i < in.size(); i++) in[i] = value(r, i, salt) + 100 * r;
      BCUDA(cudaMemcpyAsync(send[r], in.data(), in.size() * 4, cudaMemcpyHostToDevice, st));
      BCUDA(cudaMemsetAsync(recv[r], 0xEE, words * nranks * 4 + 64, st));
      BCUDA(cudaStreamSynchronize(st));
    }
    res = b200collEmuAllToAll(comms.data(), nranks, send.data(), recv.data(), per, st);
    if (res == ncclSuccess) {
      BCUDA(cudaStreamSynchronize(st));
      for (int r = 0; r < nranks; r++) {
        std::vector<int32_t> out(words * nranks + 16);
        BCUDA(cudaMemcpy(out.data(), recv[r], out.size() * 4, cudaMemcpyDeviceToHost));
        for (int src = 0; src < nranks; src++)
          for (size_t i = 0; i < words; i++)
            if (out[(size_t)src * words + i] != value(src, (size_t)r * words + i, salt) + 100 * src) (*wrong)++;
        for (size_t i = words * nranks; i < words * nranks + 16; i++)
          if ((uint32_t)out[i] != 0xEEEEEEEEu) (*wrong)++;
      }
    }
  }
  // The same exchange through the staging halves (the form for large chunks): several steps with the small staging of this test.
  if (res == ncclSuccess) {
    salt++;
    const size_t words = count;  // elements per pair
    for (int r = 0; r < nranks; r++) {
      std::vector<int32_t> in(words * nranks);
      for (size_t i = 0; i < in.size(); i++) in[i] = value(r, i, salt) + 100 * r;
      BCUDA(cudaMemcpyAsync(send[r], in.data(), in.size() * 4, cudaMemcpyHostToDevice, st));
      BCUDA(cudaMemsetAsync(recv[r], 0xEE, words * nranks * 4 + 64, st));
      BCUDA(cudaStreamSynchronize(st));
    }
    res = b200collEmuCollective(comms.data(), nranks, COLL_ALLTOALL, send.data(), recv.data(), words, ncclInt32, ncclSum, 0, 0, st);
    if (res == ncclSuccess) {
      BCUDA(cudaStreamSynchronize(st));
      const long long before = *wrong;
      for (int r = 0; r < nranks; r++) {
        std::vector<int32_t> out(words * nranks + 16);
        BCUDA(cudaMemcpy(out.data(), recv[r], out.size() * 4, cudaMemcpyDeviceToHost));
        for (int src = 0; src < nranks; src++)
          for (size_t i = 0; i < words; i++)
            if (out[(size_t)src * words + i] != value(src, (size_t)r * words + i, salt) + 100 * src) (*wrong)++;
        for (size_t i = words * nranks; i < words * nranks + 16; i++)
          if ((uint32_t)out[i] != 0xEEEEEEEEu) (*wrong)++;
      }
      if (*wrong != before) BWARN("emulated ranks: %lld wrong values in the staged all-to-all, %d ranks, %zu elements per pair", *wrong - before, nranks, count);
    }
  }
  // Device-initiated communication: put+signal ring and remote atomics, every PE a block of one kernel.
  if (res == ncclSuccess) {
    int errs = 0;
    res = b200shmem_emu_selftest(comms.data(), nranks, 4099, 4, 51, &errs);
    *wrong += errs;
  }
  for (int r = 0; r < nranks; r++) {
    ncclResult_t ae = ncclSuccess;
    tlsEmuCall = true;
    ncclCommGetAsyncError(comms[r], &ae);
    tlsEmuCall = false;
    if (ae != ncclSuccess && *status == 0) *status = (int)ae;
  }
  cudaStreamSynchronize(st);
  for (int r = 0; r < nranks; r++) {
    cudaFree(send[r]);
    cudaFree(recv[r]);
  }
  cudaStreamDestroy(st);
  for (int r = 0; r < nranks; r++) ncclCommDestroy(comms[r]);  // deferred until the last one, then torn down together
  return res;
}

}  // extern "C"
