// Public C entry points: the p-prefixed implementations, the interceptable dispatch table the
// un-prefixed names go through, group semantics, tool loading, and the extension calls.
//
// Table hand-off follows the pattern the reference's registration shim tests with its mock RCCL
// (rocprofiler-register/tests/rccl/rccl.cpp:35-126): build the table of implementations once,
// give tools one chance to wrap slots, then route every public call through it.
#include <memory>
#include <dlfcn.h>
#include <string.h>
#include <strings.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <fstream>
#include <functional>
#include <map>
#include <mutex>
#include <sstream>
#include <thread>
#include <vector>

#include "../coll/enqueue.h"
#include "../coll/launch.h"
#include "../trace/tracer.h"
#include "b200coll/api_trace.h"
#include "b200coll/nccl.h"
#include "comm.h"
#include "json.h"

using namespace b200;

namespace {

// ---- group state (per thread) ----------------------------------------------------------------
struct InitJob {
  ncclComm_t* out;
  int nranks, rank, dev;
  ncclUniqueId id;
  ncclConfig_t cfg;
  bool hasCfg;
};
struct GroupState {
  int depth = 0;
  std::vector<std::function<ncclResult_t()>> colls;
  std::vector<std::pair<Comm*, std::vector<P2pReq>>> p2p;
  std::vector<InitJob> inits;
  ncclResult_t err = ncclSuccess;
};
thread_local GroupState tlsGroup;

std::vector<P2pReq>& p2pListFor(Comm* c) {
  for (auto& kv : tlsGroup.p2p)
    if (kv.first == c) return kv.second;
  tlsGroup.p2p.emplace_back(c, std::vector<P2pReq>());
  return tlsGroup.p2p.back().second;
}

ncclResult_t runOrQueue(std::function<ncclResult_t()> fn) {
  if (tlsGroup.depth > 0) {
    tlsGroup.colls.push_back(std::move(fn));
    return ncclSuccess;
  }
  return fn();
}

// ---- schedule files (mscclLoadAlgo) -------------------------------------------------------------
struct Schedule {
  bool used = false;
  std::string name;
  int coll = -1;
  int algo = ALGO_AUTO;
  int ctas = 0;
};
std::mutex gSchedMu;
std::vector<Schedule> gSchedules;

int collFromString(const std::string& s) {
  if (s == "allreduce") return COLL_ALLREDUCE;
  if (s == "reducescatter" || s == "reduce_scatter") return COLL_REDUCESCATTER;
  if (s == "reduce") return COLL_REDUCE;
  if (s == "allgather" || s == "all_gather") return COLL_ALLGATHER;
  if (s == "broadcast") return COLL_BROADCAST;
  return -1;
}

}  // namespace

extern "C" {

// =================================================================================================
// Implementations (p-prefixed)
// =================================================================================================

ncclResult_t pncclGetVersion(int* version) {
  if (!version) BFAIL(ncclInvalidArgument, "ncclGetVersion: null pointer");
  *version = NCCL_VERSION_CODE;
  return ncclSuccess;
}

ncclResult_t pncclGetUniqueId(ncclUniqueId* id) {
  if (!id) BFAIL(ncclInvalidArgument, "ncclGetUniqueId: null pointer");
  return bootCreateRoot(id);
}

ncclResult_t pncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, ncclConfig_t* config) {
  if (!comm) BFAIL(ncclInvalidArgument, "ncclCommInitRank: null communicator pointer");
  *comm = nullptr;
  if (tlsGroup.depth > 0) {
    InitJob j{};
    j.out = comm;
    j.nranks = nranks;
    j.rank = rank;
    j.id = id;
    j.hasCfg = config != nullptr;
    if (config) j.cfg = *config;
    if (cudaGetDevice(&j.dev) != cudaSuccess) { (void)cudaGetLastError(); BFAIL(ncclUnhandledCudaError, "no CUDA device is current"); }
    tlsGroup.inits.push_back(j);
    return ncclSuccess;
  }
  Comm* c = nullptr;
  BCHECK(commCreate(&c, id, nranks, rank, config));
  *comm = reinterpret_cast<ncclComm_t>(c);
  return ncclSuccess;
}

ncclResult_t pncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank) {
  return pncclCommInitRankConfig(comm, nranks, id, rank, nullptr);
}

ncclResult_t pncclCommInitAll(ncclComm_t* comms, int ndev, const int* devlist) {
  if (!comms || ndev < 1) BFAIL(ncclInvalidArgument, "ncclCommInitAll: bad arguments");
  if (devlist && !Flags::get().emulateRanks)
    for (int i = 0; i < ndev; i++)
      for (int j = i + 1; j < ndev; j++)
        if (devlist[i] == devlist[j]) BFAIL(ncclInvalidUsage, "ncclCommInitAll: device %d appears twice", devlist[i]);
  ncclUniqueId id;
  BCHECK(bootCreateRoot(&id));
  std::vector<ncclResult_t> res(ndev, ncclSuccess);
  std::vector<std::thread> th;
  int prev = -1;
  cudaGetDevice(&prev);
  for (int i = 0; i < ndev; i++) {
    th.emplace_back([&, i] {
      int dev = devlist ? devlist[i] : i;
      if (cudaSetDevice(dev) != cudaSuccess) { (void)cudaGetLastError(); res[i] = ncclUnhandledCudaError; return; }
      Comm* c = nullptr;
      res[i] = commCreate(&c, id, ndev, i, nullptr);
      comms[i] = reinterpret_cast<ncclComm_t>(c);
    });
  }
  for (auto& t : th) t.join();
  if (prev >= 0) cudaSetDevice(prev);
  for (ncclResult_t r : res) if (r != ncclSuccess) return r;
  return ncclSuccess;
}

ncclResult_t pncclCommFinalize(ncclComm_t comm) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(c->cudaDev);
  cudaError_t e = cudaDeviceSynchronize();
  if (prev >= 0) cudaSetDevice(prev);
  if (e != cudaSuccess) { (void)cudaGetLastError(); BFAIL(ncclUnhandledCudaError, "ncclCommFinalize: %s", cudaGetErrorString(e)); }
  commPollStatus(c);
  c->finalized.store(true);
  return ncclSuccess;
}

ncclResult_t pncclCommDestroy(ncclComm_t comm) {
  if (!comm) return ncclSuccess;
  return commDestroy(asComm(comm), false);
}

ncclResult_t pncclCommAbort(ncclComm_t comm) {
  if (!comm) return ncclSuccess;
  return commDestroy(asComm(comm), true);
}

ncclResult_t pncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, ncclConfig_t* config) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!newcomm) BFAIL(ncclInvalidArgument, "ncclCommSplit: null output");
  if (color < 0 && color != NCCL_SPLIT_NOCOLOR) BFAIL(ncclInvalidArgument, "ncclCommSplit: color must be >= 0 or NCCL_SPLIT_NOCOLOR");
  *newcomm = nullptr;
  const int n = c->nranks;
  struct CK { int color, key; } mine{color, key}, all[kMaxRanks];
  BCHECK(c->boot.allGather(&mine, all, sizeof(CK)));
  // Members of my colour ordered by (key, old rank); the first is the leader and makes the id.
  std::vector<int> members;
  for (int p = 0; p < n; p++) if (color != NCCL_SPLIT_NOCOLOR && all[p].color == color) members.push_back(p);
  std::stable_sort(members.begin(), members.end(), [&](int a, int b) { return all[a].key < all[b].key; });
  ncclUniqueId myId;
  memset(&myId, 0, sizeof(myId));
  ncclResult_t leaderRes = ncclSuccess;
  if (!members.empty() && members[0] == c->rank) leaderRes = bootCreateRoot(&myId);
  std::vector<ncclUniqueId> ids(n);
  BCHECK(c->boot.allGather(&myId, ids.data(), sizeof(ncclUniqueId)));
  BCHECK(leaderRes);
  if (color == NCCL_SPLIT_NOCOLOR) return ncclSuccess;
  int newRank = (int)(std::find(members.begin(), members.end(), c->rank) - members.begin());
  ncclConfig_t cfg = config ? *config : c->config;
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(c->cudaDev);
  Comm* nc = nullptr;
  ncclResult_t r = commCreate(&nc, ids[members[0]], (int)members.size(), newRank, &cfg);
  if (prev >= 0) cudaSetDevice(prev);
  BCHECK(r);
  *newcomm = reinterpret_cast<ncclComm_t>(nc);
  return ncclSuccess;
}

const char* pncclGetErrorString(ncclResult_t r) {
  switch (r) {
    case ncclSuccess: return "no error";
    case ncclUnhandledCudaError: return "unhandled cuda error (run with NCCL_DEBUG=INFO for details)";
    case ncclSystemError: return "unhandled system error (run with NCCL_DEBUG=INFO for details)";
    case ncclInternalError: return "internal error - please report this issue to the developers";
    case ncclInvalidArgument: return "invalid argument (run with NCCL_DEBUG=WARN for details)";
    case ncclInvalidUsage: return "invalid usage (run with NCCL_DEBUG=WARN for details)";
    case ncclRemoteError: return "remote process exited or a peer stopped answering";
    case ncclInProgress: return "operation in progress";
    default: return "unknown result code";
  }
}

const char* pncclGetLastError(ncclComm_t comm) {
  Comm* c = asComm(comm);
  if (c && c->magic == kCommMagic) {
    std::lock_guard<std::mutex> lk(c->mu);
    if (!c->lastErr.empty()) {
      static thread_local std::string copy;
      copy = c->lastErr;
      return copy.c_str();
    }
  }
  return lastError();
}

ncclResult_t pncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* asyncError) {
  Comm* c = asComm(comm);
  if (!c || c->magic != kCommMagic) BFAIL(ncclInvalidArgument, "invalid communicator handle");
  if (!asyncError) BFAIL(ncclInvalidArgument, "null pointer");
  commPollStatus(c);
  *asyncError = (ncclResult_t)c->asyncError.load();
  return ncclSuccess;
}

ncclResult_t pncclCommCount(const ncclComm_t comm, int* count) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!count) BFAIL(ncclInvalidArgument, "null pointer");
  *count = c->nranks;
  return ncclSuccess;
}
ncclResult_t pncclCommCuDevice(const ncclComm_t comm, int* device) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!device) BFAIL(ncclInvalidArgument, "null pointer");
  *device = c->cudaDev;
  return ncclSuccess;
}
ncclResult_t pncclCommUserRank(const ncclComm_t comm, int* rank) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!rank) BFAIL(ncclInvalidArgument, "null pointer");
  *rank = c->rank;
  return ncclSuccess;
}

ncclResult_t pncclMemAlloc(void** ptr, size_t size) { return localAllocExportable(ptr, size); }
ncclResult_t pncclMemFree(void* ptr) { return localFreeExportable(ptr); }

ncclResult_t pncclCommRegister(const ncclComm_t comm, void* buff, size_t size, void** handle) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!buff || !size || !handle) BFAIL(ncclInvalidArgument, "ncclCommRegister: bad arguments");
  Registration* r = new Registration{buff, size};
  std::lock_guard<std::mutex> lk(c->mu);
  c->regs.push_back(r);
  *handle = r;
  return ncclSuccess;
}

ncclResult_t pncclCommDeregister(const ncclComm_t comm, void* handle) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  std::lock_guard<std::mutex> lk(c->mu);
  auto it = std::find(c->regs.begin(), c->regs.end(), (Registration*)handle);
  if (it == c->regs.end()) BFAIL(ncclInvalidArgument, "ncclCommDeregister: unknown handle");
  // The peer mapping (if one was made) stays until the communicator goes away: peers may hold it.
  delete *it;
  c->regs.erase(it);
  return ncclSuccess;
}

ncclResult_t pncclRedOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t dt, ncclScalarResidence_t residence, ncclComm_t comm) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!op || !scalar) BFAIL(ncclInvalidArgument, "ncclRedOpCreatePreMulSum: null pointer");
  if ((int)dt < 0 || (int)dt >= ncclNumTypes) BFAIL(ncclInvalidArgument, "invalid datatype %d", (int)dt);
  PreMulOp pm;
  pm.used = true;
  pm.dtype = dt;
  pm.bits = 0;
  if (residence == ncclScalarHostImmediate) memcpy(&pm.bits, scalar, dtypeSize(dt));
  else pm.devPtr = scalar;
  std::lock_guard<std::mutex> lk(c->mu);
  size_t idx = 0;
  for (; idx < c->premul.size(); idx++) if (!c->premul[idx].used) break;
  if (idx == c->premul.size()) c->premul.push_back(pm);
  else c->premul[idx] = pm;
  *op = (ncclRedOp_t)((int)ncclNumOps + (int)idx);
  return ncclSuccess;
}

ncclResult_t pncclRedOpDestroy(ncclRedOp_t op, ncclComm_t comm) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  int idx = (int)op - (int)ncclNumOps;
  std::lock_guard<std::mutex> lk(c->mu);
  if ((int)op < (int)ncclNumOps) BFAIL(ncclInvalidArgument, "ncclRedOpDestroy: %d is a built-in operator", (int)op);
  if (idx < 0 || idx >= (int)c->premul.size() || !c->premul[idx].used) BFAIL(ncclInvalidArgument, "ncclRedOpDestroy: unknown operator %d", (int)op);
  c->premul[idx].used = false;
  return ncclSuccess;
}

// ---- collectives -------------------------------------------------------------------------------
static ncclResult_t coll(int apiId, int kind, const void* send, void* recv, size_t count, ncclDataType_t dt, int op, int root, ncclComm_t comm, cudaStream_t s) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  CollReq r{};
  r.apiId = apiId;
  r.kind = kind;
  r.send = send;
  r.recv = recv;
  r.count = count;
  r.dt = dt;
  r.op = op;
  r.root = root;
  r.comm = c;
  r.stream = s;
  return runOrQueue([r] { return enqueueColl(r); });
}

ncclResult_t pncclAllReduce(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclRedOp_t op, ncclComm_t comm, cudaStream_t s) {
  return coll(B200COLL_API_ID_ncclAllReduce, COLL_ALLREDUCE, send, recv, count, dt, (int)op, 0, comm, s);
}
ncclResult_t pncclReduceScatter(const void* send, void* recv, size_t recvcount, ncclDataType_t dt, ncclRedOp_t op, ncclComm_t comm, cudaStream_t s) {
  return coll(B200COLL_API_ID_ncclReduceScatter, COLL_REDUCESCATTER, send, recv, recvcount, dt, (int)op, 0, comm, s);
}
ncclResult_t pncclAllGather(const void* send, void* recv, size_t sendcount, ncclDataType_t dt, ncclComm_t comm, cudaStream_t s) {
  return coll(B200COLL_API_ID_ncclAllGather, COLL_ALLGATHER, send, recv, sendcount, dt, ncclSum, 0, comm, s);
}
ncclResult_t pncclBroadcast(const void* send, void* recv, size_t count, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t s) {
  return coll(B200COLL_API_ID_ncclBroadcast, COLL_BROADCAST, send, recv, count, dt, ncclSum, root, comm, s);
}
ncclResult_t pncclBcast(void* buff, size_t count, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t s) {
  return coll(B200COLL_API_ID_ncclBroadcast, COLL_BROADCAST, buff, buff, count, dt, ncclSum, root, comm, s);
}
ncclResult_t pncclReduce(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclRedOp_t op, int root, ncclComm_t comm, cudaStream_t s) {
  return coll(B200COLL_API_ID_ncclReduce, COLL_REDUCE, send, recv, count, dt, (int)op, root, comm, s);
}

// ---- point-to-point and what is built on it -------------------------------------------------------
static ncclResult_t p2pOne(int apiId, bool isSend, const void* buf, size_t count, ncclDataType_t dt, int peer, ncclComm_t comm, cudaStream_t s) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if ((int)dt < 0 || (int)dt >= ncclNumTypes) BFAIL(ncclInvalidArgument, "invalid datatype %d", (int)dt);
  if (peer < 0 || peer >= c->nranks) BFAIL(ncclInvalidArgument, "peer %d outside [0, %d)", peer, c->nranks);
  if (count && !buf) BFAIL(ncclInvalidArgument, "null buffer");
  P2pReq q{isSend, const_cast<void*>(buf), count * dtypeSize(dt), peer, s, apiId};
  if (tlsGroup.depth > 0) {
    p2pListFor(c).push_back(q);
    return ncclSuccess;
  }
  std::vector<P2pReq> one{q};
  return enqueueP2pGroup(c, one);
}

ncclResult_t pncclSend(const void* send, size_t count, ncclDataType_t dt, int peer, ncclComm_t comm, cudaStream_t s) {
  return p2pOne(B200COLL_API_ID_ncclSend, true, send, count, dt, peer, comm, s);
}
ncclResult_t pncclRecv(void* recv, size_t count, ncclDataType_t dt, int peer, ncclComm_t comm, cudaStream_t s) {
  return p2pOne(B200COLL_API_ID_ncclRecv, false, recv, count, dt, peer, comm, s);
}

ncclResult_t pncclGroupStart(void);
ncclResult_t pncclGroupEnd(void);

ncclResult_t pncclAllToAll(const void* send, void* recv, size_t count, ncclDataType_t dt, ncclComm_t comm, cudaStream_t s) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (send == recv && count) BFAIL(ncclInvalidUsage, "ncclAllToAll cannot run in place");
  const size_t es = dtypeSize(dt);
  if (!es) BFAIL(ncclInvalidArgument, "invalid datatype %d", (int)dt);
  const size_t chunk = count * es;
  // Small chunks: one kernel over the flag-in-data buffers (no credits, no barrier).
  if (tlsGroup.depth == 0 && !Flags::get().emulateRanks && llAllToAllFits(c, chunk))
    return enqueueLLAllToAll(c, B200COLL_API_ID_ncclAllToAll, send, recv, count, dt, s);
  // Large chunks in ordinary buffers: peer stores into the staging halves, one barrier per step (see A2A_STAGED_MIN).
  auto stagedWanted = [&]() {
    const long long lim = Flags::get().a2aStagedMin;
    if (lim >= 0) return chunk >= (size_t)lim;
    return chunk >= ((size_t)1 << 20);   // measured between two GPUs: 1.2 - 1.5x NCCL at 8 - 128 MiB per pair where the FIFOs gave 0.85 - 1.05
  };
  // Receive buffer inside a symmetric window (the same place on every rank), whole 16-byte units: peer stores, one kernel.
  if (c->nranks > 1 && tlsGroup.depth == 0 && chunk && (chunk & 15) == 0 && ((((uintptr_t)send) | ((uintptr_t)recv)) & 15) == 0 && !Flags::get().emulateRanks) {
    if (!c->regs.empty()) BCHECK(commRegisterLazy(c, recv, 1));
    size_t off = 0;
    Window* w = nullptr;
    {
      std::lock_guard<std::mutex> lk(c->mu);
      w = c->findWindow(recv, chunk * c->nranks, &off);
    }
    if (w) {
      if (c->asyncError.load() != ncclSuccess) BFAIL((ncclResult_t)c->asyncError.load(), "communicator is in an error state: %s", c->lastErr.c_str());
      A2aDirectArgs a{};
      a.send = (const char*)send;
      for (int p = 0; p < c->nranks; p++) a.recvPeer[p] = w->seg.peer[p] + off;
      a.chunkBytes = chunk;
      int prev = -1;
      cudaGetDevice(&prev);
      if (prev != c->cudaDev) cudaSetDevice(c->cudaDev);
      Tracer* tr = c->tracer;
      TraceStamp* stamp = tr ? tr->begin(B200COLL_API_ID_ncclAllToAll, dt, count, chunk * c->nranks) : nullptr;
      DevComm dc = c->dev;
      dc.opSeq = ++c->opSeq;
      dc.stamp = stamp;
      const size_t want = (chunk * c->nranks + (256u << 10) - 1) / (256u << 10);  // one CTA per 256 KiB moved
      const int ctas = (int)std::max<size_t>(1, std::min<size_t>(want, (size_t)c->maxCtas));
      if (tr) tr->setAlgo(ALGO_P2P, ctas);
      cudaError_t e = launchAllToAllDirect(ctas, s, dc, a);
      if (tr) tr->end(e == cudaSuccess);
      if (prev != c->cudaDev && prev >= 0) cudaSetDevice(prev);
      if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "all-to-all launch failed: %s", cudaGetErrorString(e));
      return ncclSuccess;
    }
  }
  if (c->nranks > 1 && tlsGroup.depth == 0 && chunk && !Flags::get().emulateRanks && stagedWanted())
    return enqueueStagedAllToAll(c, B200COLL_API_ID_ncclAllToAll, send, recv, count, dt, s);
  pncclGroupStart();
  ncclResult_t r = ncclSuccess;
  for (int p = 0; p < c->nranks && r == ncclSuccess; p++) {
    r = p2pOne(B200COLL_API_ID_ncclAllToAll, true, (const char*)send + (size_t)p * count * es, count, dt, p, comm, s);
    if (r == ncclSuccess) r = p2pOne(B200COLL_API_ID_ncclAllToAll, false, (char*)recv + (size_t)p * count * es, count, dt, p, comm, s);
  }
  ncclResult_t e = pncclGroupEnd();
  return r != ncclSuccess ? r : e;
}

ncclResult_t pncclAllToAllv(const void* send, const size_t sendcounts[], const size_t sdispls[], void* recv, const size_t recvcounts[],
                            const size_t rdispls[], ncclDataType_t dt, ncclComm_t comm, cudaStream_t s) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!sendcounts || !sdispls || !recvcounts || !rdispls) BFAIL(ncclInvalidArgument, "ncclAllToAllv: null count/displacement array");
  const size_t es = dtypeSize(dt);
  if (!es) BFAIL(ncclInvalidArgument, "invalid datatype %d", (int)dt);
  pncclGroupStart();
  ncclResult_t r = ncclSuccess;
  for (int p = 0; p < c->nranks && r == ncclSuccess; p++) {
    r = p2pOne(B200COLL_API_ID_ncclAllToAllv, true, (const char*)send + sdispls[p] * es, sendcounts[p], dt, p, comm, s);
    if (r == ncclSuccess) r = p2pOne(B200COLL_API_ID_ncclAllToAllv, false, (char*)recv + rdispls[p] * es, recvcounts[p], dt, p, comm, s);
  }
  ncclResult_t e = pncclGroupEnd();
  return r != ncclSuccess ? r : e;
}

ncclResult_t pncclGather(const void* send, void* recv, size_t sendcount, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t s) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (root < 0 || root >= c->nranks) BFAIL(ncclInvalidArgument, "root %d outside [0, %d)", root, c->nranks);
  const size_t es = dtypeSize(dt);
  if (!es) BFAIL(ncclInvalidArgument, "invalid datatype %d", (int)dt);
  pncclGroupStart();
  ncclResult_t r = p2pOne(B200COLL_API_ID_ncclGather, true, send, sendcount, dt, root, comm, s);
  if (c->rank == root)
    for (int p = 0; p < c->nranks && r == ncclSuccess; p++)
      r = p2pOne(B200COLL_API_ID_ncclGather, false, (char*)recv + (size_t)p * sendcount * es, sendcount, dt, p, comm, s);
  ncclResult_t e = pncclGroupEnd();
  return r != ncclSuccess ? r : e;
}

ncclResult_t pncclScatter(const void* send, void* recv, size_t recvcount, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t s) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (root < 0 || root >= c->nranks) BFAIL(ncclInvalidArgument, "root %d outside [0, %d)", root, c->nranks);
  const size_t es = dtypeSize(dt);
  if (!es) BFAIL(ncclInvalidArgument, "invalid datatype %d", (int)dt);
  pncclGroupStart();
  ncclResult_t r = ncclSuccess;
  if (c->rank == root)
    for (int p = 0; p < c->nranks && r == ncclSuccess; p++)
      r = p2pOne(B200COLL_API_ID_ncclScatter, true, (const char*)send + (size_t)p * recvcount * es, recvcount, dt, p, comm, s);
  if (r == ncclSuccess) r = p2pOne(B200COLL_API_ID_ncclScatter, false, recv, recvcount, dt, root, comm, s);
  ncclResult_t e = pncclGroupEnd();
  return r != ncclSuccess ? r : e;
}

// ---- schedule files ---------------------------------------------------------------------------
ncclResult_t pmscclLoadAlgo(const char* path, mscclAlgoHandle_t* handle, int rank) {
  (void)rank;
  if (!path || !handle) BFAIL(ncclInvalidArgument, "mscclLoadAlgo: null argument");
  std::ifstream f(path);
  if (!f) BFAIL(ncclSystemError, "mscclLoadAlgo: cannot read '%s'", path);
  std::stringstream ss;
  ss << f.rdbuf();
  std::string text = ss.str();
  JsonValue root;
  JsonParser p(text);
  if (!p.parse(&root) || root.kind != JsonValue::Object) BFAIL(ncclInvalidArgument, "mscclLoadAlgo: '%s' is not a JSON schedule", path);
  Schedule sch;
  sch.used = true;
  sch.name = root.stringOr("name", path);
  sch.coll = collFromString(root.stringOr("coll", ""));
  if (sch.coll < 0) BFAIL(ncclInvalidArgument, "mscclLoadAlgo: schedule names no supported collective");
  std::string a = root.stringOr("algo", "auto");
  sch.algo = a == "ll" ? ALGO_LL : a == "p2p" ? ALGO_P2P : a == "nvls" ? ALGO_NVLS : ALGO_AUTO;
  sch.ctas = (int)root.numberOr("ctas", 0);
  std::lock_guard<std::mutex> lk(gSchedMu);
  size_t i = 0;
  for (; i < gSchedules.size(); i++) if (!gSchedules[i].used) break;
  if (i == gSchedules.size()) gSchedules.push_back(sch);
  else gSchedules[i] = sch;
  *handle = (mscclAlgoHandle_t)i;
  return ncclSuccess;
}

ncclResult_t pmscclRunAlgo(const void* send, const size_t sendCounts[], const size_t sDisPls[], void* recv, const size_t recvCounts[],
                           const size_t rDisPls[], size_t count, ncclDataType_t dt, int root, int peer, ncclRedOp_t op,
                           mscclAlgoHandle_t handle, ncclComm_t comm, cudaStream_t s) {
  (void)sendCounts; (void)sDisPls; (void)recvCounts; (void)rDisPls; (void)peer;
  Schedule sch;
  {
    std::lock_guard<std::mutex> lk(gSchedMu);
    if (handle < 0 || handle >= (int)gSchedules.size() || !gSchedules[handle].used) BFAIL(ncclInvalidArgument, "mscclRunAlgo: unknown schedule %d", handle);
    sch = gSchedules[handle];
  }
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  CollReq r{};
  r.apiId = B200COLL_API_ID_mscclRunAlgo;
  r.kind = sch.coll;
  r.send = send;
  r.recv = recv;
  r.count = count;
  r.dt = dt;
  r.op = (int)op;
  r.root = root;
  r.comm = c;
  r.stream = s;
  r.forceAlgo = sch.algo;
  r.forceCtas = sch.ctas;
  return runOrQueue([r] { return enqueueColl(r); });
}

ncclResult_t pmscclUnloadAlgo(mscclAlgoHandle_t handle) {
  std::lock_guard<std::mutex> lk(gSchedMu);
  if (handle < 0 || handle >= (int)gSchedules.size() || !gSchedules[handle].used) BFAIL(ncclInvalidArgument, "mscclUnloadAlgo: unknown schedule %d", handle);
  gSchedules[handle].used = false;
  return ncclSuccess;
}

// ---- groups ------------------------------------------------------------------------------------
ncclResult_t pncclGroupStart(void) {
  tlsGroup.depth++;
  return ncclSuccess;
}

ncclResult_t pncclGroupEnd(void) {
  if (tlsGroup.depth == 0) BFAIL(ncclInvalidUsage, "ncclGroupEnd without ncclGroupStart");
  if (--tlsGroup.depth > 0) return ncclSuccess;
  GroupState g = std::move(tlsGroup);
  tlsGroup = GroupState();
  ncclResult_t res = ncclSuccess;
  // Communicator creation blocks on the rendezvous, so grouped inits run side by side.
  if (!g.inits.empty()) {
    std::vector<ncclResult_t> rs(g.inits.size(), ncclSuccess);
    std::vector<std::thread> th;
    for (size_t i = 0; i < g.inits.size(); i++) {
      th.emplace_back([&, i] {
        InitJob& j = g.inits[i];
        if (cudaSetDevice(j.dev) != cudaSuccess) { (void)cudaGetLastError(); rs[i] = ncclUnhandledCudaError; return; }
        Comm* c = nullptr;
        rs[i] = commCreate(&c, j.id, j.nranks, j.rank, j.hasCfg ? &j.cfg : nullptr);
        *j.out = reinterpret_cast<ncclComm_t>(c);
      });
    }
    for (auto& t : th) t.join();
    for (ncclResult_t r : rs) if (r != ncclSuccess && res == ncclSuccess) res = r;
  }
  for (auto& fn : g.colls) {
    ncclResult_t r = fn();
    if (r != ncclSuccess && res == ncclSuccess) res = r;
  }
  for (auto& kv : g.p2p) {
    ncclResult_t r = enqueueP2pGroup(kv.first, kv.second);
    if (r != ncclSuccess && res == ncclSuccess) res = r;
  }
  return res;
}

// =================================================================================================
// Dispatch table and tool loading
// =================================================================================================

static b200collApiFuncTable gTable;
static std::once_flag gTableOnce;

// Secure mode (B200COLL_TOOL_SECURE=1): a tool library is code that runs inside every rank, so only libraries named by an
// absolute path, owned by root or by this user and writable by nobody else are loaded, and a tool symbol that merely happens
// to be in the process is not trusted. B200COLL_TOOL_REGISTER_ENABLED=0 switches tool loading off altogether. The reference's
// registration shim has the same two switches (rocprofiler-register README: ROCPROFILER_REGISTER_ENABLED, _SECURE).
static bool trustedToolFile(const std::string& path, std::string* why) {
  if (path.empty() || path[0] != '/') { *why = "not an absolute path"; return false; }
  struct stat st;
  if (stat(path.c_str(), &st) != 0 || !S_ISREG(st.st_mode)) { *why = "not a regular file"; return false; }
  if (st.st_uid != 0 && st.st_uid != geteuid()) { *why = "owned by another user"; return false; }
  if (st.st_mode & (S_IWGRP | S_IWOTH)) { *why = "writable by group or others"; return false; }
  return true;
}

static void loadTools() {
  auto on = [](const char* name, bool dflt) {
    const char* v = getenv(name);
    return (v && *v) ? (strcmp(v, "0") != 0 && strcasecmp(v, "false") != 0 && strcasecmp(v, "off") != 0) : dflt;
  };
  if (!on("B200COLL_TOOL_REGISTER_ENABLED", true)) return;
  const bool secure = on("B200COLL_TOOL_SECURE", false);
  // A tool already in the process (linked or LD_PRELOADed) …
  std::vector<b200collToolConfigure_fn> fns;
  if (!secure)
    if (void* sym = dlsym(RTLD_DEFAULT, "b200coll_tool_configure")) fns.push_back((b200collToolConfigure_fn)sym);
  // … and every library named in B200COLL_TOOL_LIBRARIES.
  const std::string& libs = Flags::get().toolLibs;
  size_t pos = 0;
  while (pos < libs.size()) {
    size_t c = libs.find(':', pos);
    std::string one = libs.substr(pos, c == std::string::npos ? std::string::npos : c - pos);
    pos = c == std::string::npos ? libs.size() : c + 1;
    if (one.empty()) continue;
    std::string why;
    if (secure && !trustedToolFile(one, &why)) {
      BWARN("tool library '%s' refused in secure mode: %s", one.c_str(), why.c_str());
      continue;
    }
    void* h = dlopen(one.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) {
      BWARN("tool library '%s' could not be loaded: %s", one.c_str(), dlerror());
      continue;
    }
    void* sym = dlsym(h, "b200coll_tool_configure");
    if (!sym) {
      BWARN("tool library '%s' has no b200coll_tool_configure", one.c_str());
      continue;
    }
    if (std::find(fns.begin(), fns.end(), (b200collToolConfigure_fn)sym) == fns.end()) fns.push_back((b200collToolConfigure_fn)sym);
  }
  const uint32_t ver = B200COLL_API_TRACE_VERSION_MAJOR * 10000 + B200COLL_API_TRACE_VERSION_PATCH;
  uint64_t id = 1;
  for (auto fn : fns) {
    int rc = fn(ver, &gTable, id++);
    if (rc != 0) BWARN("a tool's b200coll_tool_configure returned %d", rc);
  }
}

static void buildTable() {
  gTable.size = sizeof(gTable);
#define B200_SLOT(name) gTable.name##_fn = p##name;
  B200_SLOT(ncclAllGather) B200_SLOT(ncclAllReduce) B200_SLOT(ncclAllToAll) B200_SLOT(ncclAllToAllv) B200_SLOT(ncclBroadcast)
  B200_SLOT(ncclGather) B200_SLOT(ncclReduce) B200_SLOT(ncclReduceScatter) B200_SLOT(ncclScatter) B200_SLOT(ncclSend) B200_SLOT(ncclRecv)
  B200_SLOT(ncclRedOpCreatePreMulSum) B200_SLOT(ncclRedOpDestroy) B200_SLOT(ncclGroupStart) B200_SLOT(ncclGroupEnd) B200_SLOT(ncclGetVersion)
  B200_SLOT(ncclGetUniqueId) B200_SLOT(ncclCommInitRank) B200_SLOT(ncclCommInitAll) B200_SLOT(ncclCommInitRankConfig) B200_SLOT(ncclCommFinalize)
  B200_SLOT(ncclCommDestroy) B200_SLOT(ncclCommAbort) B200_SLOT(ncclCommSplit) B200_SLOT(ncclGetErrorString) B200_SLOT(ncclGetLastError)
  B200_SLOT(ncclCommGetAsyncError) B200_SLOT(ncclCommCount) B200_SLOT(ncclCommCuDevice) B200_SLOT(ncclCommUserRank) B200_SLOT(ncclMemAlloc)
  B200_SLOT(ncclMemFree) B200_SLOT(mscclLoadAlgo) B200_SLOT(mscclRunAlgo) B200_SLOT(mscclUnloadAlgo) B200_SLOT(ncclCommRegister)
  B200_SLOT(ncclCommDeregister)
#undef B200_SLOT
  loadTools();
}

b200collApiFuncTable* b200collGetApiTable(void) {
  std::call_once(gTableOnce, buildTable);
  return &gTable;
}

// The ABI promise of api_trace.h: `size`, then one pointer per slot in id order.
static_assert(sizeof(b200collApiFuncTable) == 8 + 8 * B200COLL_API_ID_LAST, "dispatch table layout changed");
static_assert(offsetof(b200collApiFuncTable, ncclAllGather_fn) == 8 + 8 * B200COLL_API_ID_ncclAllGather, "slot moved");
static_assert(offsetof(b200collApiFuncTable, ncclRecv_fn) == 8 + 8 * B200COLL_API_ID_ncclRecv, "slot moved");
static_assert(offsetof(b200collApiFuncTable, ncclCommSplit_fn) == 8 + 8 * B200COLL_API_ID_ncclCommSplit, "slot moved");
static_assert(offsetof(b200collApiFuncTable, ncclMemFree_fn) == 8 + 8 * B200COLL_API_ID_ncclMemFree, "slot moved");
static_assert(offsetof(b200collApiFuncTable, ncclCommDeregister_fn) == 8 + 8 * B200COLL_API_ID_ncclCommDeregister, "slot moved");

#define T() b200collGetApiTable()
ncclResult_t ncclMemAlloc(void** ptr, size_t size) { return T()->ncclMemAlloc_fn(ptr, size); }
ncclResult_t ncclMemFree(void* ptr) { return T()->ncclMemFree_fn(ptr); }
ncclResult_t ncclGetVersion(int* v) { return T()->ncclGetVersion_fn(v); }
ncclResult_t ncclGetUniqueId(ncclUniqueId* id) { return T()->ncclGetUniqueId_fn(id); }
ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int n, ncclUniqueId id, int rank, ncclConfig_t* cfg) { return T()->ncclCommInitRankConfig_fn(comm, n, id, rank, cfg); }
ncclResult_t ncclCommInitRank(ncclComm_t* comm, int n, ncclUniqueId id, int rank) { return T()->ncclCommInitRank_fn(comm, n, id, rank); }
ncclResult_t ncclCommInitAll(ncclComm_t* comm, int ndev, const int* devlist) { return T()->ncclCommInitAll_fn(comm, ndev, devlist); }
ncclResult_t ncclCommFinalize(ncclComm_t comm) { return T()->ncclCommFinalize_fn(comm); }
ncclResult_t ncclCommDestroy(ncclComm_t comm) { return T()->ncclCommDestroy_fn(comm); }
ncclResult_t ncclCommAbort(ncclComm_t comm) { return T()->ncclCommAbort_fn(comm); }
ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, ncclConfig_t* cfg) { return T()->ncclCommSplit_fn(comm, color, key, newcomm, cfg); }
const char* ncclGetErrorString(ncclResult_t r) { return T()->ncclGetErrorString_fn(r); }
const char* ncclGetLastError(ncclComm_t comm) { return T()->ncclGetLastError_fn(comm); }
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* e) { return T()->ncclCommGetAsyncError_fn(comm, e); }
ncclResult_t ncclCommCount(const ncclComm_t comm, int* count) { return T()->ncclCommCount_fn(comm, count); }
ncclResult_t ncclCommCuDevice(const ncclComm_t comm, int* dev) { return T()->ncclCommCuDevice_fn(comm, dev); }
ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank) { return T()->ncclCommUserRank_fn(comm, rank); }
ncclResult_t ncclCommRegister(const ncclComm_t comm, void* buff, size_t size, void** handle) { return T()->ncclCommRegister_fn(comm, buff, size, handle); }
ncclResult_t ncclCommDeregister(const ncclComm_t comm, void* handle) { return T()->ncclCommDeregister_fn(comm, handle); }
ncclResult_t ncclRedOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t dt, ncclScalarResidence_t res, ncclComm_t comm) { return T()->ncclRedOpCreatePreMulSum_fn(op, scalar, dt, res, comm); }
ncclResult_t ncclRedOpDestroy(ncclRedOp_t op, ncclComm_t comm) { return T()->ncclRedOpDestroy_fn(op, comm); }
ncclResult_t ncclReduce(const void* s, void* r, size_t c, ncclDataType_t dt, ncclRedOp_t op, int root, ncclComm_t comm, cudaStream_t st) { return T()->ncclReduce_fn(s, r, c, dt, op, root, comm, st); }
ncclResult_t ncclBcast(void* b, size_t c, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t st) { return T()->ncclBroadcast_fn(b, b, c, dt, root, comm, st); }
ncclResult_t ncclBroadcast(const void* s, void* r, size_t c, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t st) { return T()->ncclBroadcast_fn(s, r, c, dt, root, comm, st); }
ncclResult_t ncclAllReduce(const void* s, void* r, size_t c, ncclDataType_t dt, ncclRedOp_t op, ncclComm_t comm, cudaStream_t st) { return T()->ncclAllReduce_fn(s, r, c, dt, op, comm, st); }
ncclResult_t ncclReduceScatter(const void* s, void* r, size_t c, ncclDataType_t dt, ncclRedOp_t op, ncclComm_t comm, cudaStream_t st) { return T()->ncclReduceScatter_fn(s, r, c, dt, op, comm, st); }
ncclResult_t ncclAllGather(const void* s, void* r, size_t c, ncclDataType_t dt, ncclComm_t comm, cudaStream_t st) { return T()->ncclAllGather_fn(s, r, c, dt, comm, st); }
ncclResult_t ncclSend(const void* s, size_t c, ncclDataType_t dt, int peer, ncclComm_t comm, cudaStream_t st) { return T()->ncclSend_fn(s, c, dt, peer, comm, st); }
ncclResult_t ncclRecv(void* r, size_t c, ncclDataType_t dt, int peer, ncclComm_t comm, cudaStream_t st) { return T()->ncclRecv_fn(r, c, dt, peer, comm, st); }
ncclResult_t ncclGather(const void* s, void* r, size_t c, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t st) { return T()->ncclGather_fn(s, r, c, dt, root, comm, st); }
ncclResult_t ncclScatter(const void* s, void* r, size_t c, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t st) { return T()->ncclScatter_fn(s, r, c, dt, root, comm, st); }
ncclResult_t ncclAllToAll(const void* s, void* r, size_t c, ncclDataType_t dt, ncclComm_t comm, cudaStream_t st) { return T()->ncclAllToAll_fn(s, r, c, dt, comm, st); }
ncclResult_t ncclAllToAllv(const void* s, const size_t sc[], const size_t sd[], void* r, const size_t rc[], const size_t rd[], ncclDataType_t dt, ncclComm_t comm, cudaStream_t st) { return T()->ncclAllToAllv_fn(s, sc, sd, r, rc, rd, dt, comm, st); }
ncclResult_t mscclLoadAlgo(const char* path, mscclAlgoHandle_t* h, int rank) { return T()->mscclLoadAlgo_fn(path, h, rank); }
ncclResult_t mscclRunAlgo(const void* s, const size_t sc[], const size_t sd[], void* r, const size_t rc[], const size_t rd[], size_t c, ncclDataType_t dt, int root, int peer, ncclRedOp_t op, mscclAlgoHandle_t h, ncclComm_t comm, cudaStream_t st) { return T()->mscclRunAlgo_fn(s, sc, sd, r, rc, rd, c, dt, root, peer, op, h, comm, st); }
ncclResult_t mscclUnloadAlgo(mscclAlgoHandle_t h) { return T()->mscclUnloadAlgo_fn(h); }
ncclResult_t ncclGroupStart(void) { return T()->ncclGroupStart_fn(); }
ncclResult_t ncclGroupEnd(void) { return T()->ncclGroupEnd_fn(); }
#undef T

// =================================================================================================
// Extensions
// =================================================================================================

ncclResult_t b200collSymAlloc(ncclComm_t comm, size_t size, void** ptr) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!ptr || !size) BFAIL(ncclInvalidArgument, "b200collSymAlloc: bad arguments");
  return commSymAlloc(c, size, ptr);
}
ncclResult_t b200collSymFree(ncclComm_t comm, void* ptr) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  return commSymFree(c, ptr);
}
ncclResult_t b200collSymPeerPtr(ncclComm_t comm, const void* ptr, int peer, void** peerPtr) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!peerPtr || peer < 0 || peer >= c->nranks) BFAIL(ncclInvalidArgument, "b200collSymPeerPtr: bad arguments");
  size_t off = 0;
  std::lock_guard<std::mutex> lk(c->mu);
  Window* w = c->findWindow(ptr, 1, &off);
  if (!w) BFAIL(ncclInvalidArgument, "%p is not inside a symmetric allocation of this communicator", ptr);
  *peerPtr = w->seg.peer[peer] + off;
  return ncclSuccess;
}
ncclResult_t b200collSymMulticastPtr(ncclComm_t comm, const void* ptr, void** mcPtr) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!mcPtr) BFAIL(ncclInvalidArgument, "b200collSymMulticastPtr: null output");
  size_t off = 0;
  std::lock_guard<std::mutex> lk(c->mu);
  Window* w = c->findWindow(ptr, 1, &off);
  if (!w) BFAIL(ncclInvalidArgument, "%p is not inside a symmetric allocation of this communicator", ptr);
  *mcPtr = w->seg.mc ? w->seg.mc + off : nullptr;
  return ncclSuccess;
}
ncclResult_t b200collHostBarrier(ncclComm_t comm) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  return c->boot.barrier();
}
ncclResult_t b200collHostAllGather(ncclComm_t comm, const void* send, void* recv, size_t bytes) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  return c->boot.allGather(send, recv, bytes);
}
ncclResult_t b200collBarrier(ncclComm_t comm, cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (c->nranks == 1) return ncclSuccess;
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != c->cudaDev) cudaSetDevice(c->cudaDev);
  DevComm dc = c->dev;
  dc.opSeq = ++c->opSeq;
  cudaError_t e = launchBarrier(stream, dc);
  if (prev != c->cudaDev && prev >= 0) cudaSetDevice(prev);
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "barrier launch failed: %s", cudaGetErrorString(e));
  return ncclSuccess;
}

ncclResult_t b200collTraceEnable(ncclComm_t comm, int on) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (on && !c->tracer) c->tracer = new Tracer(c->rank, c->nranks, c->cudaDev);
  if (!on && c->tracer) {
    c->tracer->drain();
    delete c->tracer;
    c->tracer = nullptr;
  }
  return ncclSuccess;
}
ncclResult_t b200collTraceGet(ncclComm_t comm, b200collTraceRecordC* out, size_t max, size_t* n) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!n) BFAIL(ncclInvalidArgument, "null pointer");
  if (!c->tracer) { *n = 0; return ncclSuccess; }
  c->tracer->drain();
  *n = c->tracer->copyOut(out, max);
  return ncclSuccess;
}
ncclResult_t b200collTraceDropped(ncclComm_t comm, uint64_t* dropped) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!dropped) BFAIL(ncclInvalidArgument, "null pointer");
  *dropped = c->tracer ? c->tracer->dropped() : 0;
  return ncclSuccess;
}
ncclResult_t b200collTraceClear(ncclComm_t comm) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (c->tracer) c->tracer->clear();
  return ncclSuccess;
}
ncclResult_t b200collTraceWrite(ncclComm_t comm, const char* path, const char* format) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  if (!c->tracer || !path) BFAIL(ncclInvalidUsage, "tracing is not enabled on this communicator");
  c->tracer->drain();
  bool ok = (format && strcmp(format, "perfetto") == 0) ? c->tracer->writePerfetto(path) : c->tracer->writeCsv(path);
  if (!ok) BFAIL(ncclSystemError, "cannot write trace to '%s'", path);
  return ncclSuccess;
}

}  // extern "C"

// ---- host-only rendezvous handles (used by tests and by the Python layer without a GPU) ---------
extern "C" {
// What the planner would choose for a collective on a communicator of `nranks` ranks, with or without
// a multicast alias, without any device or peer: the algorithm (1 flag-in-data, 2 peer loads, 3 in-switch),
// CTAs, whether the zero-copy path applies (never here: the buffers are not in a window) and the number of
// pipeline chunks. Honours the environment and the tuning file exactly as a real communicator does.
// `kind`: 0 all-reduce, 1 reduce-scatter, 2 reduce, 3 all-gather, 4 broadcast, 5 all-to-all (count per pair; algorithm 4 = send/recv FIFOs).
ncclResult_t b200collPlanDry(int nranks, int nvls, int kind, size_t count, ncclDataType_t dt, ncclRedOp_t op, b200collPlanInfo* out) {
  if (!out || nranks < 1 || nranks > kMaxRanks || kind < 0 || kind > COLL_ALLTOALL || (int)dt < 0 || (int)dt >= ncclNumTypes)
    BFAIL(ncclInvalidArgument, "b200collPlanDry: bad argument");
  const Flags& fl = Flags::get();
  auto c = std::make_unique<Comm>();
  c->magic = kCommMagic;
  c->rank = 0;
  c->nranks = nranks;
  c->nvls = nvls != 0 && fl.nvlsEnable != 0 && nranks > 1;
  c->dev.rank = 0;
  c->dev.nranks = nranks;
  c->dev.stageBytes = nranks == 1 ? (1u << 16) : fl.stageBytes;
  if (fl.maxCtas > 0) c->maxCtas = fl.maxCtas;
  if (fl.minCtas > 0) c->minCtas = fl.minCtas;
  if (c->maxCtas > kMaxCtas) c->maxCtas = kMaxCtas;
  if (c->minCtas > c->maxCtas) c->minCtas = c->maxCtas;
  loadTuning(c.get());
  if (kind == COLL_ALLTOALL) {
    // `count` elements per pair, as ncclAllToAll decides (ordinary buffers): 1 flag-in-data kernel, 2 staged kernel by peer
    // stores (chunks = its steps), 4 grouped send/recv over the FIFOs.
    const size_t chunk = count * dtypeSize(dt);
    out->direct = 0;
    if (nranks == 1 || chunk == 0) {
      out->algo = ALGO_P2P; out->ctas = 1; out->chunks = 1;
    } else if (llAllToAllFits(c.get(), chunk)) {
      out->algo = ALGO_LL;
      out->ctas = std::max(1, std::min((int)((chunk / 8 + kCollThreads - 1) / kCollThreads), std::min(llCtaCap(chunk, nranks), std::max(16, c->maxCtas))));
      out->chunks = 0;
    } else if (fl.a2aStagedMin >= 0 ? chunk >= (size_t)fl.a2aStagedMin : chunk >= ((size_t)1 << 20)) {
      CollArgs args;
      DevComm dc;
      int ctas = 0;
      stagedAllToAllArgs(c.get(), nullptr, nullptr, count, dt, 0, &args, &dc, &ctas);
      out->algo = ALGO_P2P; out->ctas = ctas; out->chunks = c->stageParity;
    } else {
      out->algo = 4; out->ctas = 0; out->chunks = (chunk + fl.p2pChunkBytes - 1) / fl.p2pChunkBytes;
    }
    return ncclSuccess;
  }
  CollReq r{};
  r.kind = kind;
  r.send = reinterpret_cast<const void*>(0x10000);  // never dereferenced on the host; aligned, outside any window
  r.recv = reinterpret_cast<void*>(0x20000);
  r.count = count;
  r.dt = dt;
  r.op = (int)op;
  r.root = 0;
  r.comm = c.get();
  Plan plan{};
  BCHECK(planColl(r, &plan));
  out->algo = plan.algo;
  out->ctas = plan.ctas;
  out->direct = plan.direct ? 1 : 0;
  out->chunks = plan.chunks;
  return ncclSuccess;
}

// Copies the JSON description of every setting into `buf` (NUL-terminated, truncated to `cap`);
// returns the length the full text needs.
size_t b200collDescribeSettings(char* buf, size_t cap) {
  const std::string s = describeSettings();
  if (buf && cap) {
    const size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
    memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return s.size() + 1;
}

ncclResult_t b200collBootCreate(const ncclUniqueId* id, int rank, int nranks, void** handle) {
  if (!id || !handle) BFAIL(ncclInvalidArgument, "b200collBootCreate: null argument");
  Bootstrap* b = new Bootstrap();
  ncclResult_t r = b->init(*id, rank, nranks);
  if (r != ncclSuccess) { delete b; *handle = nullptr; return r; }
  *handle = b;
  return ncclSuccess;
}
ncclResult_t b200collBootAllGather(void* handle, const void* send, void* recv, size_t bytes) {
  if (!handle) BFAIL(ncclInvalidArgument, "null bootstrap handle");
  return ((Bootstrap*)handle)->allGather(send, recv, bytes);
}
ncclResult_t b200collBootBarrier(void* handle) {
  if (!handle) BFAIL(ncclInvalidArgument, "null bootstrap handle");
  return ((Bootstrap*)handle)->barrier();
}
ncclResult_t b200collBootSendFd(void* handle, int peer, int fd, uint32_t tag) {
  if (!handle) BFAIL(ncclInvalidArgument, "null bootstrap handle");
  return ((Bootstrap*)handle)->sendFd(peer, fd, tag);
}
ncclResult_t b200collBootRecvFd(void* handle, int peer, uint32_t tag, int* fd) {
  if (!handle || !fd) BFAIL(ncclInvalidArgument, "null argument");
  return ((Bootstrap*)handle)->recvFd(peer, tag, fd);
}
int b200collBootPeerFailed(void* handle) {
  int who = -1;
  if (!handle) return -1;
  return ((Bootstrap*)handle)->peerFailed(&who) ? who : -1;
}
ncclResult_t b200collBootClose(void* handle, int graceful) {
  if (!handle) return ncclSuccess;
  Bootstrap* b = (Bootstrap*)handle;
  b->close(graceful != 0);
  delete b;
  return ncclSuccess;
}
void b200collRefreshFlags(void) { Flags::refresh(); }
// Enqueue a wait on a flag nothing sets, with `timeoutMs` as its budget (test hook for the
// time-out path; the communicator reports ncclRemoteError afterwards and must be destroyed).
ncclResult_t b200collTestWaitTimeout(ncclComm_t comm, int timeoutMs, cudaStream_t stream) {
  Comm* c = asComm(comm);
  BCHECK(commCheck(c));
  DevComm dc = c->dev;
  dc.opSeq = ++c->opSeq;
  dc.timeoutNs = (unsigned long long)timeoutMs * 1000000ull;
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != c->cudaDev) cudaSetDevice(c->cudaDev);
  cudaError_t e = launchWaitUnsetFlag(stream, dc);
  if (prev != c->cudaDev && prev >= 0) cudaSetDevice(prev);
  if (e != cudaSuccess) BFAIL(ncclUnhandledCudaError, "launch failed: %s", cudaGetErrorString(e));
  return ncclSuccess;
}
// What the communicator was able to set up: bit 0 multicast (NVLS), bit 1 legacy IPC mode.
int b200collCommCaps(ncclComm_t comm) {
  Comm* c = asComm(comm);
  if (!c || c->magic != kCommMagic) return -1;
  return (c->nvls ? 1 : 0) | (c->ws.legacy ? 2 : 0);
}
const char* b200collLastError(void) { return lastError(); }
}
