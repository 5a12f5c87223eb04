#include "enqueue.h"

#include <string.h>

#include <algorithm>

#include "../trace/tracer.h"
#include "b200coll/api_trace.h"
#include "launch.h"

namespace b200 {

// Flag-in-data kernels: up to 16 CTAs for the latency-bound sizes; beyond that one per 16 KiB of the message past 256 KiB,
// or one per 64 KiB of lines a rank stores into its peers (2 x bytes x (n - 1): between eight ranks a CTA of a 256 KiB
// all-reduce would otherwise store 224 KiB of lines by itself), whichever is more, up to 64.
int llCtaCap(size_t bytes, int nranks) {
  const int bySize = bytes <= (256u << 10) ? 16 : std::min(64, std::max(16, (int)(bytes >> 14)));
  const size_t stored = bytes * 2 * (size_t)std::max(1, nranks - 1);
  return std::max(bySize, (int)std::min<size_t>(64, stored >> 16));
}

namespace {

struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) {
      cudaSetDevice(dev);
      switched = true;
    }
  }
  ~DeviceGuard() {
    if (switched && prev >= 0) cudaSetDevice(prev);
  }
};

struct ResolvedOp {
  int base;          // ncclSum/Prod/Max/Min
  int scaleMode;
  unsigned long long bits;
  const void* devPtr = nullptr;  // PreMulSum scalar that lives in device memory: the kernel reads it
};

ncclResult_t resolveOp(Comm* c, int op, ncclDataType_t dt, ResolvedOp* out) {
  out->bits = 0;
  out->devPtr = nullptr;
  out->scaleMode = SCALE_NONE;
  if (op >= 0 && op < ncclNumOps) {
    if (op == ncclAvg) {
      out->base = ncclSum;
      out->scaleMode = SCALE_POST_DIV_N;
    } else {
      out->base = op;
    }
    return ncclSuccess;
  }
  int idx = op - (int)ncclNumOps;
  PreMulOp pm;
  {
    std::lock_guard<std::mutex> lk(c->mu);
    if (idx < 0 || idx >= (int)c->premul.size() || !c->premul[idx].used) BFAIL(ncclInvalidArgument, "reduction operator %d does not exist on this communicator", op);
    pm = c->premul[idx];
  }
  if (pm.dtype != dt) BFAIL(ncclInvalidArgument, "PreMulSum operator was created for %s, used with %s", dtypeName(pm.dtype), dtypeName(dt));
  out->base = ncclSum;
  out->scaleMode = SCALE_PRE_MUL;
  // A scalar in device memory is read by the kernel, in stream order: no host wait, and the call can be captured.
  out->devPtr = pm.devPtr;
  out->bits = pm.bits;
  return ncclSuccess;
}

int ctasFor(const Comm* c, size_t bytes, int algo) {
  // Mid-size messages are bound by NVLink latency, not bandwidth, so they want many CTAs with
  // little work each: one CTA per 64 KiB (128 KiB on the in-switch path, whose loads are wider
  // per instruction), between the communicator's bounds.
  size_t per = algo == ALGO_NVLS ? (128u << 10) : (64u << 10);
  size_t want = (bytes + per - 1) / per;
  int hi = c->maxCtas;
  int ctas = (int)std::min<size_t>(want, (size_t)hi);
  return std::max(ctas, c->minCtas);
}

bool findTuning(const Comm* c, int kind, size_t bytes, int* algo, int* ctas) {
  for (const TuneEntry& t : c->tuning) {
    if (t.coll >= 0 && t.coll != kind) continue;
    if (bytes > t.maxBytes) continue;
    *algo = t.algo;
    *ctas = t.ctas;
    return true;
  }
  return false;
}

size_t traceBytes(const CollReq& r) {
  size_t b = r.count * dtypeSize(r.dt);
  if (r.kind == COLL_ALLGATHER || r.kind == COLL_REDUCESCATTER) b *= r.comm->nranks;
  return b;
}

}  // namespace

static ncclResult_t planInternal(const CollReq& r, const ResolvedOp& rop, Plan* plan, CollArgs* args) {
  Comm* c = r.comm;
  const int n = c->nranks;
  const size_t es = dtypeSize(r.dt);
  const size_t bytes = r.count * es;  // per-rank slice for RS/AG
  const Flags& fl = Flags::get();
  const bool reducing = r.kind == COLL_ALLREDUCE || r.kind == COLL_REDUCESCATTER || r.kind == COLL_REDUCE;

  int algo = r.forceAlgo, ctas = r.forceCtas;
  if (algo == ALGO_AUTO) {
    int ta = ALGO_AUTO, tc = 0;
    if (findTuning(c, r.kind, bytes, &ta, &tc)) {
      algo = ta;
      if (!ctas) ctas = tc;
    }
  }
  if (algo == ALGO_AUTO && !fl.algo.empty()) {
    if (fl.algo == "ll") algo = ALGO_LL;
    else if (fl.algo == "p2p" || fl.algo == "simple" || fl.algo == "ring" || fl.algo == "tree") algo = ALGO_P2P;
    else if (fl.algo == "nvls") algo = ALGO_NVLS;
  }
  const bool nvlsOk = c->nvls && n > 1 && (!reducing || (nvlsReducible(r.dt, rop.base) && rop.scaleMode != SCALE_PRE_MUL)) &&
                      (r.kind == COLL_ALLREDUCE || r.kind == COLL_REDUCESCATTER || r.kind == COLL_REDUCE || r.kind == COLL_BROADCAST);
  const bool llOk = n > 1 && ((r.kind == COLL_ALLREDUCE && bytes <= fl.llLimit(n)) ||
                             ((r.kind == COLL_REDUCESCATTER || r.kind == COLL_ALLGATHER) && bytes <= fl.llSliceLimit(n)));
  if (algo == ALGO_LL && !llOk) algo = ALGO_AUTO;
  if (algo == ALGO_NVLS && !nvlsOk) algo = ALGO_AUTO;
  const bool builtinChoice = algo == ALGO_AUTO;
  if (algo == ALGO_AUTO) {
    // In-switch reduction moves S(1 + 1/n) bytes per GPU and direction for an all-reduce of S
    // bytes (every rank's copy goes to the switch, the requester's own included) against
    // 2S(n-1)/n with peer loads and stores: a win from four ranks up, a loss between two.
    // A broadcast between two ranks is one plain store stream into the peer's staging (measured: 0.95 - 1.0 of NCCL at
    // 8 MiB - 512 MiB, against 0.79 - 0.95 through the multicast address, which also writes the root's own replica).
    const bool nvlsPays = n > 2;
    if (llOk) algo = ALGO_LL;
    else if (nvlsOk && nvlsPays && bytes * (r.kind == COLL_REDUCESCATTER ? n : 1) >= (32u << 10)) algo = ALGO_NVLS;
    else algo = ALGO_P2P;
  }

  memset(args, 0, sizeof(*args));
  args->send = r.send;
  args->recv = r.recv;
  args->count = r.count;
  args->kind = r.kind;
  args->root = r.root;
  args->scaleMode = rop.scaleMode;
  args->scalarBits = rop.bits;
  args->scalarPtr = rop.devPtr;

  // Zero-copy windows: buffers inside symmetric allocations (b200collSymAlloc, or ncclMemAlloc +
  // ncclCommRegister) are read and written in place on every rank.
  bool direct = false;
  // Reduce with peer loads would need the root's recv window on ranks that may pass no recv.
  // PreMulSum scales inputs while staging them, so it cannot skip staging.
  const bool directKind = !(r.kind == COLL_REDUCE && algo != ALGO_NVLS) && rop.scaleMode != SCALE_PRE_MUL;
  plan->sendWin = plan->recvWin = 0;
  plan->sendOff = plan->recvOff = 0;
  if (algo != ALGO_LL && n > 1 && (bytes % 16) == 0 && directKind && r.allowDirect) {
    const size_t sendBytes = r.kind == COLL_REDUCESCATTER ? bytes * n : bytes;
    const size_t recvBytes = r.kind == COLL_ALLGATHER ? bytes * n : bytes;
    const bool needSend = r.kind != COLL_BROADCAST;
    const bool needRecv = r.kind == COLL_ALLREDUCE || r.kind == COLL_BROADCAST;
    size_t so = 0, ro = 0;
    Window* sw = nullptr;
    Window* rw = nullptr;
    {
      std::lock_guard<std::mutex> lk(c->mu);
      if (needSend && r.send) sw = c->findWindow(r.send, sendBytes, &so);
      if (needRecv && r.recv) rw = c->findWindow(r.recv, recvBytes, &ro);
    }
    const bool aligned = ((((uintptr_t)(needSend ? r.send : nullptr)) | ((uintptr_t)r.recv)) & 15) == 0;
    const bool mcOk = (!needSend || (sw && sw->seg.mc)) && (!needRecv || (rw && rw->seg.mc));
    const bool mcNeeded = algo == ALGO_NVLS;
    if (aligned && (!needSend || sw) && (!needRecv || rw) && (!mcNeeded || mcOk)) {
      direct = true;
      plan->sendWin = sw ? sw->id : 0;
      plan->recvWin = rw ? rw->id : 0;
      plan->sendOff = so;
      plan->recvOff = ro;
      for (int p = 0; p < n; p++) {
        args->sendPeer[p] = sw ? sw->seg.peer[p] + so : nullptr;
        args->recvPeer[p] = rw ? rw->seg.peer[p] + ro : nullptr;
      }
      args->sendMc = sw && sw->seg.mc ? sw->seg.mc + so : nullptr;
      args->recvMc = rw && rw->seg.mc ? rw->seg.mc + ro : nullptr;
    }
  }
  args->direct = direct ? 1 : 0;
  // A large broadcast through staging goes by peer stores (scatter and forward: every link carries each byte once, pipelined
  // over the staging halves). One multicast store stream from the root tops out near 400 GB/s (eight GPUs: 0.58 - 0.68 of
  // NCCL from 128 MiB; the scatter-and-forward form measured 0.81 at 512 MiB between four); up to one staging half the
  // multicast form has fewer barriers and measured 0.9 - 1.4. It also stays the way into symmetric windows, where the
  // alternative would be n - 1 store streams from the root.
  if (builtinChoice && r.kind == COLL_BROADCAST && algo == ALGO_NVLS && !direct && bytes > c->dev.stageBytes) algo = ALGO_P2P;

  size_t chunks = 0;
  args->chunkBytes = 0;
  if (algo != ALGO_LL && !direct) {
    const bool reduceKind = r.kind == COLL_ALLREDUCE || r.kind == COLL_REDUCESCATTER || r.kind == COLL_REDUCE;
    const size_t fullCap = r.kind == COLL_REDUCESCATTER ? ((c->dev.stageBytes / n) & ~(size_t)15) : c->dev.stageBytes;
    size_t capMax = fullCap;
    if (reduceKind && fl.pipeChunkBytes != 0) {
      // Pipeline chunk of the reducing kernels: an eighth of what moves through staging, between
      // 32 MiB and one staging half. A chunk costs its inter-rank barriers (about 8 us measured between
      // two GPUs): with 8 MiB chunks a 32 MiB all-reduce took 107 us, as one chunk 83 us, and every size
      // up to 256 MiB was fastest with 32 MiB chunks.
      const size_t staged = r.kind == COLL_REDUCESCATTER ? bytes * n : bytes;
      if (staged > (size_t)32 << 20 || fl.pipeChunkBytes > 0) {
        size_t chunk = std::max<size_t>((size_t)32 << 20, ((staged / 8) + ((1u << 20) - 1)) & ~(size_t)((1u << 20) - 1));
        if (fl.pipeChunkBytes > 0) chunk = ((size_t)fl.pipeChunkBytes + 4095) & ~(size_t)4095;
        const size_t perCall = r.kind == COLL_REDUCESCATTER ? (chunk / n) & ~(size_t)15 : chunk;
        if (perCall >= 16 && perCall < capMax) capMax = perCall;
      }
    }
    // Equal chunks: the kernels place data in staging by the chunk capacity alone, so a short
    // last chunk would leave most lanes idle.
    const size_t k = (bytes + capMax - 1) / capMax;
    size_t cap = (((bytes + k - 1) / k) + 15) & ~(size_t)15;  // k == 1: the message itself, so every lane gets a share
    if (cap > capMax) cap = capMax;
    if (cap < fullCap) args->chunkBytes = cap;
    chunks = (bytes + cap - 1) / cap;
  }
  if (!ctas) {
    size_t moved = bytes * ((r.kind == COLL_REDUCESCATTER || r.kind == COLL_ALLGATHER) ? n : 1);
    ctas = algo == ALGO_LL ? (int)((bytes / 8 + kCollThreads - 1) / kCollThreads) : ctasFor(c, moved, algo);
  }
  const int llCap = llCtaCap(bytes, n);
  ctas = std::max(1, std::min(ctas, algo == ALGO_LL ? std::min(llCap, std::max(16, c->maxCtas)) : c->maxCtas));
  plan->algo = algo;
  plan->ctas = ctas;
  plan->direct = direct;
  plan->chunks = chunks;
  return ncclSuccess;
}

ncclResult_t planColl(const CollReq& r, Plan* plan) {
  ResolvedOp rop{ncclSum, SCALE_NONE, 0};
  if (r.op >= 0 && r.op < ncclNumOps) {
    rop.base = r.op == ncclAvg ? ncclSum : r.op;
    rop.scaleMode = r.op == ncclAvg ? SCALE_POST_DIV_N : SCALE_NONE;
  } else {
    rop.scaleMode = SCALE_PRE_MUL;
  }
  CollArgs args;
  return planInternal(r, rop, plan, &args);
}

ncclResult_t emuPrepare(const CollReq& r, Plan* plan, CollArgs* args, LLArgs* ll, DevComm* dc) {
  Comm* c = r.comm;
  BCHECK(commCheck(c));
  const int n = c->nranks;
  if ((int)r.dt < 0 || (int)r.dt >= ncclNumTypes) BFAIL(ncclInvalidArgument, "invalid datatype %d", (int)r.dt);
  if (r.op < 0 || r.op >= ncclNumOps) BFAIL(ncclInvalidArgument, "the emulation takes the built-in reduction operators only");
  if (n < 2 || r.count == 0) BFAIL(ncclInvalidArgument, "the emulation needs at least two ranks and a non-empty message");
  const bool rooted = r.kind == COLL_REDUCE || r.kind == COLL_BROADCAST;
  if (rooted && (r.root < 0 || r.root >= n)) BFAIL(ncclInvalidArgument, "root %d outside [0, %d)", r.root, n);
  const size_t es = dtypeSize(r.dt);
  if ((((uintptr_t)r.send) | ((uintptr_t)r.recv)) & (es - 1)) BFAIL(ncclInvalidArgument, "buffer not aligned to its element size");
  ResolvedOp rop{r.op == ncclAvg ? (int)ncclSum : r.op, r.op == ncclAvg ? SCALE_POST_DIV_N : SCALE_NONE, 0};
  BCHECK(planInternal(r, rop, plan, args));
  *dc = c->dev;
  dc->opSeq = ++c->opSeq;
  dc->stamp = nullptr;
  memset(ll, 0, sizeof(*ll));
  if (plan->algo == ALGO_LL) {
    ll->send = r.send;
    ll->recv = r.recv;
    ll->kind = r.kind;
    ll->count = r.kind == COLL_ALLGATHER ? r.count * es : r.count;
    ll->scaleMode = rop.scaleMode;
    ll->scalarBits = rop.bits;
    if (++c->llSeq == 0) c->llSeq = 2;
    ll->seq = c->llSeq;
  } else {
    args->stageHalf = (int)(c->stageParity & 1);
    c->stageParity += (uint32_t)plan->chunks;
  }
  return ncclSuccess;
}

ncclResult_t enqueueColl(const CollReq& r) {
  Comm* c = r.comm;
  BCHECK(commCheck(c));
  const int n = c->nranks;
  if ((int)r.dt < 0 || (int)r.dt >= ncclNumTypes) BFAIL(ncclInvalidArgument, "invalid datatype %d", (int)r.dt);
  const bool reducing = r.kind == COLL_ALLREDUCE || r.kind == COLL_REDUCESCATTER || r.kind == COLL_REDUCE;
  const bool rooted = r.kind == COLL_REDUCE || r.kind == COLL_BROADCAST;
  if (rooted && (r.root < 0 || r.root >= n)) BFAIL(ncclInvalidArgument, "root %d outside [0, %d)", r.root, n);
  if (c->asyncError.load() != ncclSuccess) BFAIL((ncclResult_t)c->asyncError.load(), "communicator is in an error state: %s", c->lastErr.c_str());
  if (r.count == 0) return ncclSuccess;
  const bool needRecv = !(r.kind == COLL_REDUCE && c->rank != r.root);
  const bool needSend = !(r.kind == COLL_BROADCAST && c->rank != r.root);
  if ((needSend && !r.send) || (needRecv && !r.recv)) BFAIL(ncclInvalidArgument, "null buffer");
  const size_t es = dtypeSize(r.dt);
  if ((((uintptr_t)r.send) | ((uintptr_t)r.recv)) & (es - 1)) BFAIL(ncclInvalidArgument, "buffer not aligned to its element size");

  DeviceGuard guard(c->cudaDev);
  ResolvedOp rop{ncclSum, SCALE_NONE, 0};
  if (reducing) BCHECK(resolveOp(c, r.op, r.dt, &rop));

  Tracer* tr = c->tracer;
  TraceStamp* stamp = tr ? tr->begin(r.apiId, r.dt, r.count, traceBytes(r)) : nullptr;
  auto finish = [&](bool launched, ncclResult_t res) {
    if (tr) tr->end(launched);
    return res;
  };

  // One rank: a copy, unless the operator rescales.
  if (n == 1 && rop.scaleMode != SCALE_PRE_MUL) {
    if (r.send != r.recv) {
      cudaError_t e = cudaMemcpyAsync(r.recv, r.send, r.count * es, cudaMemcpyDeviceToDevice, r.stream);
      if (e != cudaSuccess) return finish(false, ncclUnhandledCudaError);
    }
    return finish(false, ncclSuccess);
  }

  // Registered buffers are exchanged with the peers on first use.
  if (!c->regs.empty()) {
    if (r.send) BCHECK(commRegisterLazy(c, r.send, 1));
    if (r.recv) BCHECK(commRegisterLazy(c, r.recv, 1));
  }

  Plan plan;
  CollArgs args;
  BCHECK(planInternal(r, rop, &plan, &args));
  if (Flags::get().checkSymmetric && n > 1 && plan.algo != ALGO_LL) {
    // The zero-copy path applies this rank's window offsets to every peer's mapping, so it is only right when all ranks
    // passed the same place of the same window. Compare, and stage everywhere unless everybody agrees.
    struct Where { uint64_t direct, sendWin, recvWin, sendOff, recvOff; } mine{plan.direct ? 1u : 0u, plan.sendWin, plan.recvWin, plan.sendOff, plan.recvOff};
    std::vector<Where> all(n);
    BCHECK(c->boot.allGather(&mine, all.data(), sizeof(Where)));
    bool same = true;
    for (int p = 0; p < n; p++) same = same && memcmp(&all[p], &all[0], sizeof(Where)) == 0;
    if (!same || !all[0].direct) {
      if (plan.direct) BINFO(SUB_COLL, "rank %d: buffers are in a symmetric window, but not at the same place on every rank: staging", c->rank);
      CollReq staged = r;
      staged.allowDirect = false;
      BCHECK(planInternal(staged, rop, &plan, &args));
    }
  }
  DevComm dc = c->dev;
  dc.opSeq = ++c->opSeq;
  dc.stamp = stamp;
  if (tr) tr->setAlgo(plan.algo, plan.ctas);
  BTRACE(SUB_COLL, "rank %d op#%llu kind %d count %zu %s algo %d ctas %d direct %d", c->rank, (unsigned long long)dc.opSeq, r.kind, r.count, dtypeName(r.dt), plan.algo, plan.ctas, (int)plan.direct);

  cudaError_t e;
  if (plan.algo == ALGO_LL) {
    LLArgs la{};
    la.send = r.send;
    la.recv = r.recv;
    la.kind = r.kind;
    la.count = r.kind == COLL_ALLGATHER ? r.count * es : r.count;
    la.scaleMode = rop.scaleMode;
    la.scalarBits = rop.bits;
    la.scalarPtr = rop.devPtr;
    if (++c->llSeq == 0) c->llSeq = 2;  // 0 is the "never written" value; keep the parity sequence
    la.seq = c->llSeq;
    e = r.kind == COLL_ALLGATHER ? launchLLAllGather(plan.ctas, r.stream, dc, la) : launchLLAllReduce(r.dt, rop.base, plan.ctas, r.stream, dc, la);
  } else {
    args.stageHalf = (int)(c->stageParity & 1);
    c->stageParity += (uint32_t)plan.chunks;
    const bool nvls = plan.algo == ALGO_NVLS;
    // Reducing kernels run 256-thread CTAs, so twice as many for the same thread count.
    if (reducing) e = launchStagedReduce(r.dt, rop.base, nvls, std::min(2 * plan.ctas, kMaxCtas), r.stream, dc, args);
    else e = launchStagedCopy(nvls && r.kind == COLL_BROADCAST, plan.ctas, r.stream, dc, args, (int)es);
  }
  if (e != cudaSuccess) {
    setLastError("kernel launch failed: %s", cudaGetErrorString(e));
    BWARN("kernel launch failed: %s", cudaGetErrorString(e));
    return finish(false, ncclUnhandledCudaError);
  }
  return finish(true, ncclSuccess);
}

// All-to-all of small chunks through the flag-in-data buffers: one launch, no FIFO credits, no barrier. The caller has
// checked that bytesPerPeer fits (llAllToAllFits).
bool llAllToAllFits(Comm* c, size_t bytesPerPeer) {
  return c->nranks > 1 && bytesPerPeer > 0 && bytesPerPeer <= Flags::get().llSliceLimit(c->nranks);
}

ncclResult_t enqueueLLAllToAll(Comm* c, int apiId, const void* send, void* recv, size_t count, ncclDataType_t dt, cudaStream_t stream) {
  BCHECK(commCheck(c));
  if (c->asyncError.load() != ncclSuccess) BFAIL((ncclResult_t)c->asyncError.load(), "communicator is in an error state: %s", c->lastErr.c_str());
  if (!send || !recv) BFAIL(ncclInvalidArgument, "null buffer");
  const size_t bytes = count * dtypeSize(dt);
  DeviceGuard guard(c->cudaDev);
  Tracer* tr = c->tracer;
  TraceStamp* stamp = tr ? tr->begin(apiId, dt, count, bytes * c->nranks) : nullptr;
  DevComm dc = c->dev;
  dc.opSeq = ++c->opSeq;
  dc.stamp = stamp;
  LLArgs la{};
  la.send = send;
  la.recv = recv;
  la.kind = COLL_ALLTOALL;
  la.count = bytes;
  if (++c->llSeq == 0) c->llSeq = 2;
  la.seq = c->llSeq;
  const int llCap = llCtaCap(bytes, c->nranks);
  const int ctas = std::max(1, std::min((int)((bytes / 8 + kCollThreads - 1) / kCollThreads), std::min(llCap, std::max(16, c->maxCtas))));
  if (tr) tr->setAlgo(ALGO_LL, ctas);
  cudaError_t e = launchLLAllGather(ctas, stream, dc, la);
  if (tr) tr->end(e == cudaSuccess);
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "all-to-all launch failed: %s", cudaGetErrorString(e));
  return ncclSuccess;
}

// Arguments of the staged all-to-all for one rank: steps and staging parity as the kernel walks them. forceCtas: 0 = by size.
void stagedAllToAllArgs(Comm* c, const void* send, void* recv, size_t count, ncclDataType_t dt, int forceCtas, CollArgs* args, DevComm* dc, int* ctas) {
  const size_t bytes = count * dtypeSize(dt);
  const int n = c->nranks;
  *dc = c->dev;
  dc->opSeq = ++c->opSeq;
  dc->stamp = nullptr;
  memset(args, 0, sizeof(*args));
  args->send = send;
  args->recv = recv;
  args->count = count;
  args->kind = COLL_ALLTOALL;
  const size_t slotCap = (c->dev.stageBytes / (size_t)n) & ~(size_t)15;
  const size_t cap = std::min(slotCap, (bytes + 15) & ~(size_t)15);
  const size_t steps = (bytes + cap - 1) / cap;
  args->stageHalf = (int)(c->stageParity & 1);
  c->stageParity += (uint32_t)steps;
  *ctas = forceCtas > 0 ? forceCtas : std::max(1, std::min(ctasFor(c, bytes * n, ALGO_P2P), c->maxCtas));
}

// All-to-all of large chunks through the staging halves (kStagedCopy, kind COLL_ALLTOALL): peer stores into per-source
// slots, one barrier per step, local copy-out. count: elements per pair.
ncclResult_t enqueueStagedAllToAll(Comm* c, int apiId, const void* send, void* recv, size_t count, ncclDataType_t dt, cudaStream_t stream) {
  BCHECK(commCheck(c));
  if (c->asyncError.load() != ncclSuccess) BFAIL((ncclResult_t)c->asyncError.load(), "communicator is in an error state: %s", c->lastErr.c_str());
  if (!send || !recv) BFAIL(ncclInvalidArgument, "null buffer");
  const size_t es = dtypeSize(dt), bytes = count * es;
  const int n = c->nranks;
  DeviceGuard guard(c->cudaDev);
  Tracer* tr = c->tracer;
  TraceStamp* stamp = tr ? tr->begin(apiId, dt, count, bytes * n) : nullptr;
  DevComm dc;
  CollArgs args;
  int ctas = 0;
  stagedAllToAllArgs(c, send, recv, count, dt, 0, &args, &dc, &ctas);
  dc.stamp = stamp;
  if (tr) tr->setAlgo(ALGO_P2P, ctas);
  cudaError_t e = launchStagedCopy(false, ctas, stream, dc, args, (int)es);
  if (tr) tr->end(e == cudaSuccess);
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "all-to-all launch failed: %s", cudaGetErrorString(e));
  return ncclSuccess;
}

ncclResult_t enqueueP2pGroup(Comm* c, std::vector<P2pReq>& ops) {
  BCHECK(commCheck(c));
  if (ops.empty()) return ncclSuccess;
  if (c->asyncError.load() != ncclSuccess) BFAIL((ncclResult_t)c->asyncError.load(), "communicator is in an error state: %s", c->lastErr.c_str());
  DeviceGuard guard(c->cudaDev);
  const int n = c->nranks;
  for (const P2pReq& o : ops)
    if (o.peer < 0 || o.peer >= n) BFAIL(ncclInvalidArgument, "peer %d outside [0, %d)", o.peer, n);
  cudaStream_t main = ops[0].stream;
  // Other streams used in the group join the first one for the duration of the transfers.
  std::vector<cudaStream_t> others;
  for (const P2pReq& o : ops)
    if (o.stream != main && std::find(others.begin(), others.end(), o.stream) == others.end()) others.push_back(o.stream);
  for (cudaStream_t s : others) {
    BCUDA(cudaEventRecord(c->scratchEvent, s));
    BCUDA(cudaStreamWaitEvent(main, c->scratchEvent, 0));
  }

  // Self-sends pair with self-receives in order and become local copies.
  std::vector<P2pReq*> selfSend, selfRecv;
  std::vector<P2pReq*> rest;
  for (P2pReq& o : ops) {
    if (o.peer == c->rank) (o.isSend ? selfSend : selfRecv).push_back(&o);
    else rest.push_back(&o);
  }
  if (selfSend.size() != selfRecv.size()) BFAIL(ncclInvalidUsage, "%zu sends to self but %zu receives from self in one group", selfSend.size(), selfRecv.size());
  for (size_t i = 0; i < selfSend.size(); i++) {
    if (selfSend[i]->bytes != selfRecv[i]->bytes) BFAIL(ncclInvalidUsage, "send-to-self of %zu bytes meets a receive of %zu bytes", selfSend[i]->bytes, selfRecv[i]->bytes);
    if (selfSend[i]->bytes && selfSend[i]->buf != selfRecv[i]->buf)
      BCUDA(cudaMemcpyAsync(selfRecv[i]->buf, selfSend[i]->buf, selfSend[i]->bytes, cudaMemcpyDeviceToDevice, main));
  }

  // Rounds: at most one send and one receive per peer in a launch, in the order they were made.
  std::vector<bool> done(rest.size(), false);
  size_t left = rest.size();
  while (left) {
    P2pArgs pa{};
    bool sendUsed[kMaxRanks] = {}, recvUsed[kMaxRanks] = {};
    for (size_t i = 0; i < rest.size(); i++) {
      if (done[i]) continue;
      P2pReq* o = rest[i];
      bool* used = o->isSend ? sendUsed : recvUsed;
      if (used[o->peer]) continue;
      used[o->peer] = true;
      done[i] = true;
      left--;
      if (o->bytes == 0) continue;
      P2pWork& w = pa.work[pa.nwork++];
      w.peer = o->peer;
      w.isSend = o->isSend ? 1 : 0;
      w.src = (const char*)o->buf;
      w.dst = (char*)o->buf;
      w.bytes = o->bytes;
    }
    if (pa.nwork == 0) continue;
    Tracer* tr = c->tracer;
    size_t tb = 0;
    for (int i = 0; i < pa.nwork; i++) tb += pa.work[i].bytes;
    TraceStamp* stamp = tr ? tr->begin(ops[0].apiId, ncclInt8, tb, tb) : nullptr;
    DevComm dc = c->dev;
    dc.opSeq = ++c->opSeq;
    dc.stamp = stamp;
    if (tr) tr->setAlgo(ALGO_P2P, pa.nwork * dc.p2pSubs);
    cudaError_t e = launchP2p(pa.nwork * dc.p2pSubs, main, dc, pa);
    if (tr) tr->end(e == cudaSuccess);
    if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "send/recv launch failed: %s", cudaGetErrorString(e));
  }
  for (cudaStream_t s : others) {
    BCUDA(cudaEventRecord(c->scratchEvent, main));
    BCUDA(cudaStreamWaitEvent(s, c->scratchEvent, 0));
  }
  return ncclSuccess;
}

}  // namespace b200
