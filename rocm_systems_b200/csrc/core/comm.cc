#include "comm.h"

#include <string.h>
#include <unistd.h>

#include <fstream>
#include <sstream>

#include "../coll/launch.h"
#include "../trace/tracer.h"
#include "json.h"

namespace b200 {

static size_t alignUp(size_t v, size_t a) { return (v + a - 1) / a * a; }

Window* Comm::findWindow(const void* ptr, size_t bytes, size_t* off) {
  auto it = windows.upper_bound((uintptr_t)ptr);
  if (it == windows.begin()) return nullptr;
  --it;
  Window* w = it->second.get();
  uintptr_t base = it->first;
  if ((uintptr_t)ptr + bytes > base + w->seg.size) return nullptr;
  if (off) *off = (uintptr_t)ptr - base;
  return w;
}

static int collFromName(const std::string& s) {
  if (s == "allreduce" || s == "all_reduce") return COLL_ALLREDUCE;
  if (s == "reducescatter" || s == "reduce_scatter") return COLL_REDUCESCATTER;
  if (s == "reduce") return COLL_REDUCE;
  if (s == "allgather" || s == "all_gather") return COLL_ALLGATHER;
  if (s == "broadcast") return COLL_BROADCAST;
  return -1;
}
static int algoFromName(const std::string& s) {
  if (s == "ll" || s == "oneshot") return ALGO_LL;
  if (s == "p2p" || s == "twoshot" || s == "simple") return ALGO_P2P;
  if (s == "nvls" || s == "multimem") return ALGO_NVLS;
  return ALGO_AUTO;
}

// Tuning file: {"entries":[{"coll":"allreduce","max_bytes":65536,"algo":"ll","ctas":8}, ...]}
// Rows are matched in order; the first whose coll matches (or is absent) and whose max_bytes
// is >= the message size wins.
void loadTuning(Comm* c) {
  c->tuning.clear();
  const std::string& path = Flags::get().tuningFile;
  if (path.empty()) return;
  std::ifstream f(path);
  if (!f) {
    BWARN("tuning file '%s' cannot be read; using built-in thresholds", path.c_str());
    return;
  }
  std::stringstream ss;
  ss << f.rdbuf();
  std::string text = ss.str();
  JsonValue root;
  JsonParser p(text);
  if (!p.parse(&root) || root.kind != JsonValue::Object) {
    BWARN("tuning file '%s' is not valid JSON; using built-in thresholds", path.c_str());
    return;
  }
  const JsonValue* entries = root.get("entries");
  if (!entries || entries->kind != JsonValue::Array) return;
  for (const JsonValue& e : entries->arr) {
    if (e.kind != JsonValue::Object) continue;
    TuneEntry t;
    t.coll = collFromName(e.stringOr("coll", ""));
    // Numbers come from a user's file: convert with saturation (a double outside the target's range is undefined behaviour).
    auto toSize = [](double v) -> size_t { return !(v > 0) ? 0 : (v >= 1.8e19 ? ~(size_t)0 : (size_t)v); };
    auto toInt = [](double v) -> int { return !(v > 0) ? 0 : (v >= 2e9 ? 2000000000 : (int)v); };
    t.maxBytes = e.get("max_bytes") ? toSize(e.numberOr("max_bytes", 0)) : ~(size_t)0;
    t.algo = algoFromName(e.stringOr("algo", "auto"));
    t.ctas = toInt(e.numberOr("ctas", 0));
    int nr = toInt(e.numberOr("nranks", 0));
    if (nr && nr != c->nranks) continue;
    c->tuning.push_back(t);
  }
  BINFO(SUB_TUNE, "loaded %zu tuning rows from %s", c->tuning.size(), path.c_str());
}

static void watchdogLoop(Comm* c) {
  // One progress thread per communicator: folds the device status word and bootstrap failure
  // notices into the async error (what the async-events thread does for hardware events in
  // rocr-runtime/runtime/hsa-runtime/core/runtime/runtime.cpp:1547-1738).
  while (!c->stopWatchdog.load(std::memory_order_relaxed)) {
    commPollStatus(c);
    int who = -1;
    if (c->asyncError.load() == ncclSuccess && c->boot.peerFailed(&who)) {
      c->asyncError.store(ncclRemoteError);
      {
        std::lock_guard<std::mutex> lk(c->mu);
        char buf[128];
        snprintf(buf, sizeof(buf), "rank %d left the communicator", who);
        c->lastErr = buf;
      }
      BWARN("rank %d: peer rank %d is gone; pending device waits will be ended", c->rank, who);
      if (c->abortFlag) *(volatile uint32_t*)c->abortFlag = 1;
    }
    usleep(20000);
  }
}

ncclResult_t commPollStatus(Comm* c) {
  if (!c->status) return ncclSuccess;
  volatile DevStatus* s = c->status;
  uint32_t code = s->code;
  if (code != 0 && c->asyncError.load() == ncclSuccess) {
    char buf[256];
    static const char* kinds[] = {"?", "barrier", "flag-in-data line", "send/recv data", "send/recv credit", "shmem wait", "fused-op flag"};
    snprintf(buf, sizeof(buf), "device wait %s: %s on rank %u (cta %u, expected %u, saw %u, op #%llu)",
             code == 1 ? "timed out" : "aborted", s->what < 7 ? kinds[s->what] : "?", s->peer, s->cta, s->expected, s->seen,
             (unsigned long long)s->opSeq);
    {
      std::lock_guard<std::mutex> lk(c->mu);
      c->lastErr = buf;
    }
    BWARN("rank %d: %s", c->rank, buf);
    c->asyncError.store(code == 1 ? ncclRemoteError : ncclInternalError);
  }
  return ncclSuccess;
}

thread_local bool tlsEmuCall = false;

static std::mutex gGroupsMu;
static std::map<std::string, std::weak_ptr<LocalGroup>> gGroups;  // keyed by the unique id's bytes

static std::shared_ptr<LocalGroup> joinLocalGroup(const ncclUniqueId& id) {
  const std::string key(reinterpret_cast<const char*>(&id), sizeof(id));
  std::lock_guard<std::mutex> lk(gGroupsMu);
  if (gGroups.size() > 64)  // forget communicators that are long gone
    for (auto it = gGroups.begin(); it != gGroups.end();) it = it->second.expired() ? gGroups.erase(it) : std::next(it);
  std::shared_ptr<LocalGroup> g = gGroups[key].lock();
  if (!g) {
    g = std::make_shared<LocalGroup>();
    gGroups[key] = g;
  }
  std::lock_guard<std::mutex> lg(g->mu);
  g->members++;
  return g;
}

ncclResult_t commCheck(const Comm* c) {
  if (!c || c->magic != kCommMagic) BFAIL(ncclInvalidArgument, "invalid communicator handle");
  if (c->aborted.load()) BFAIL(ncclInvalidUsage, "communicator was aborted");
  if (c->destroyRequested.load()) BFAIL(ncclInvalidUsage, "communicator was destroyed");
  // Ranks that share a GPU must never run as separate kernels that wait on one another: nothing makes them run together.
  if (c->emulated && !tlsEmuCall) BFAIL(ncclInvalidUsage, "this communicator shares its GPU with other ranks (B200COLL_EMULATE_RANKS): only the b200collEmu* entry points run on it");
  return ncclSuccess;
}

ncclResult_t commCreate(Comm** out, const ncclUniqueId& id, int nranks, int rank, const ncclConfig_t* config) {
  *out = nullptr;
  const Flags& fl = Flags::get();
  if (nranks < 1 || nranks > kMaxRanks) BFAIL(ncclInvalidArgument, "nranks %d outside [1, %d] (one NVSwitch domain)", nranks, kMaxRanks);
  if (rank < 0 || rank >= nranks) BFAIL(ncclInvalidArgument, "rank %d outside [0, %d)", rank, nranks);
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  if (config) {
    if (config->magic != 0xcafebeef) BFAIL(ncclInvalidArgument, "ncclConfig_t was not initialised with NCCL_CONFIG_INITIALIZER");
    if (config->size > sizeof(ncclConfig_t)) BFAIL(ncclInvalidArgument, "ncclConfig_t is from a newer header (%zu bytes)", config->size);
    memcpy(&cfg, config, config->size);
    if (cfg.minCTAs != NCCL_CONFIG_UNDEF_INT && cfg.maxCTAs != NCCL_CONFIG_UNDEF_INT && cfg.minCTAs > cfg.maxCTAs)
      BFAIL(ncclInvalidArgument, "config.minCTAs %d > config.maxCTAs %d", cfg.minCTAs, cfg.maxCTAs);
    if (cfg.blocking != NCCL_CONFIG_UNDEF_INT && cfg.blocking != 0 && cfg.blocking != 1) BFAIL(ncclInvalidArgument, "config.blocking must be 0 or 1");
  }
  int dev = 0;
  BCUDA(cudaGetDevice(&dev));
  BCUDA(cudaFree(0));

  std::unique_ptr<Comm> c(new Comm());
  c->magic = kCommMagic;
  c->rank = rank;
  c->nranks = nranks;
  c->cudaDev = dev;
  c->config = cfg;
  c->maxCtas = 64;  // twice that for the reducing kernels' 256-thread CTAs; measured between 2 GPUs: 1 GiB all-reduce 0.80 of NCCL at 32, 1.08 at 64
  c->minCtas = 1;
  if (fl.maxCtas > 0) c->maxCtas = fl.maxCtas;
  if (fl.minCtas > 0) c->minCtas = fl.minCtas;
  if (cfg.maxCTAs != NCCL_CONFIG_UNDEF_INT && cfg.maxCTAs > 0) c->maxCtas = cfg.maxCTAs;
  if (cfg.minCTAs != NCCL_CONFIG_UNDEF_INT && cfg.minCTAs > 0) c->minCtas = cfg.minCTAs;
  if (c->maxCtas > kMaxCtas) c->maxCtas = kMaxCtas;
  if (c->minCtas > c->maxCtas) c->minCtas = c->maxCtas;

  BCHECK(c->boot.init(id, rank, nranks));

  // No two ranks on one device (rccl.h: "Using the same device for multiple ranks … not supported").
  struct Who { char bus[32]; char host[64]; } me{}, all[kMaxRanks];
  cudaDeviceGetPCIBusId(me.bus, sizeof(me.bus), dev);
  gethostname(me.host, sizeof(me.host) - 1);
  BCHECK(c->boot.allGather(&me, all, sizeof(Who)));
  for (int p = 0; p < nranks; p++) {
    if (p != rank && strcmp(all[p].bus, me.bus) == 0 && strcmp(all[p].host, me.host) == 0) {
      if (!fl.emulateRanks) BFAIL(ncclInvalidUsage, "ranks %d and %d both use GPU %s", rank, p, me.bus);
      c->emulated = true;
    }
    if (strcmp(all[p].host, me.host) != 0) BFAIL(ncclInvalidUsage, "rank %d is on host %s, rank %d on %s: one NVSwitch box only", rank, me.host, p, all[p].host);
  }

  // Workspace layout.
  DevComm& d = c->dev;
  d.rank = rank;
  d.nranks = nranks;
  const bool solo = nranks == 1;
  d.llSlotBytes = solo ? 256 : 2 * fl.llLimit(nranks);
  const size_t llBytes = 2 * (size_t)nranks * d.llSlotBytes;
  d.stageOff = alignUp(kWsLLOff + llBytes, 1u << 16);
  d.stageBytes = solo ? (1u << 16) : fl.stageBytes;
  d.p2pOff = d.stageOff + 2 * d.stageBytes;
  d.p2pChunkBytes = solo ? 4096 : fl.p2pChunkBytes;
  // Few peers: more CTAs per peer so a pair of GPUs can still fill its links.
  d.p2pSubs = fl.p2pCtasPerPeer > 0 ? fl.p2pCtasPerPeer : (nranks <= 2 ? 16 : (nranks <= 4 ? 8 : 4));
  d.p2pSlots = 4;
  const size_t p2pBytes = (size_t)nranks * d.p2pSubs * d.p2pSlots * d.p2pChunkBytes;
  const size_t total = d.p2pOff + p2pBytes;
  BCHECK(symAlloc(c->boot, dev, total, true, c->symTag, &c->ws));
  c->symTag += 2;
  for (int p = 0; p < nranks; p++) d.ws[p] = c->ws.peer[p];
  d.wsMc = c->ws.mc;
  c->nvls = c->ws.mc != nullptr;

  BCUDA(cudaMemset(c->ws.peer[rank], 0, d.stageOff));  // flags and flag-in-data lines start at zero
  BCUDA(cudaMalloc(&c->local, sizeof(LocalState)));
  BCUDA(cudaMemset(c->local, 0, sizeof(LocalState)));
  void* host = nullptr;
  BCUDA(cudaHostAlloc(&host, 256, cudaHostAllocMapped | cudaHostAllocPortable));
  memset(host, 0, 256);
  c->status = (DevStatus*)host;
  c->abortFlag = (uint32_t*)((char*)host + 128);
  void* devView = nullptr;
  BCUDA(cudaHostGetDevicePointer(&devView, host, 0));
  d.local = c->local;
  d.status = (DevStatus*)devView;
  d.abortFlag = (volatile uint32_t*)((char*)devView + 128);
  d.timeoutNs = (unsigned long long)fl.waitTimeoutMs * 1000000ull;
  d.stamp = nullptr;
  BCUDA(cudaEventCreateWithFlags(&c->scratchEvent, cudaEventDisableTiming));
  BCUDA(cudaDeviceSynchronize());
  BCHECK(c->boot.barrier());  // nobody may touch a peer's flags before they are zeroed

  loadTuning(c.get());
  if (fl.traceEnable) c->tracer = new Tracer(rank, nranks, dev);
  c->watchdog = std::thread(watchdogLoop, c.get());
  c->localGroup = joinLocalGroup(id);
  BINFO(SUB_INIT, "rank %d/%d on cuda:%d ready: workspace %zu MiB, nvls %d, ctas [%d,%d]", rank, nranks, dev, total >> 20, (int)c->nvls, c->minCtas, c->maxCtas);
  *out = c.release();
  return ncclSuccess;
}

static ncclResult_t commDestroyNow(Comm* c, bool abort);

ncclResult_t commDestroy(Comm* c, bool abort) {
  if (!c || c->magic != kCommMagic) BFAIL(ncclInvalidArgument, "invalid communicator handle");
  if (c->destroyRequested.exchange(true)) return ncclSuccess;  // already on its way out
  std::shared_ptr<LocalGroup> g = c->localGroup;
  if (!g) return commDestroyNow(c, abort);
  std::vector<Comm*> run;
  {
    std::lock_guard<std::mutex> lk(g->mu);
    if (abort) {
      g->members--;  // an aborted rank takes no part in the collective teardown of the others
    } else {
      g->waiting.push_back(c);
    }
    if (g->members > 0 && (int)g->waiting.size() >= g->members) {
      run.swap(g->waiting);
      g->members = 0;
    } else if (!abort) {
      return ncclSuccess;  // deferred: runs when the last rank of this process is destroyed
    }
  }
  ncclResult_t res = abort ? commDestroyNow(c, true) : ncclSuccess;
  if (run.size() == 1) {
    ncclResult_t r = commDestroyNow(run[0], false);
    return res != ncclSuccess ? res : r;
  }
  std::vector<ncclResult_t> rs(run.size(), ncclSuccess);
  std::vector<std::thread> th;
  for (size_t i = 0; i < run.size(); i++) th.emplace_back([&, i] { rs[i] = commDestroyNow(run[i], false); });
  for (auto& t : th) t.join();
  for (ncclResult_t r : rs)
    if (res == ncclSuccess && r != ncclSuccess) res = r;
  return res;
}

static ncclResult_t commDestroyNow(Comm* c, bool abort) {
  int prevDev = -1;
  cudaGetDevice(&prevDev);
  cudaSetDevice(c->cudaDev);
  if (abort) {
    c->aborted.store(true);
    if (c->abortFlag) *(volatile uint32_t*)c->abortFlag = 1;  // ends every device-side wait
  }
  cudaDeviceSynchronize();
  (void)cudaGetLastError();
  c->stopWatchdog.store(true);
  if (c->watchdog.joinable()) c->watchdog.join();
  if (c->tracer) {
    const std::string& tf = Flags::get().traceFile;
    if (!tf.empty()) {
      char path[512];
      snprintf(path, sizeof(path), "%s.rank%d.csv", tf.c_str(), c->rank);
      c->tracer->drain();
      c->tracer->writeCsv(path);
    }
    delete c->tracer;
    c->tracer = nullptr;
  }
  if (!abort) c->boot.barrier();  // peers may still be reading our memory until they get here
  notifyRelease(c, nullptr);
  for (auto& kv : c->windows) symFree(&kv.second->seg, c->cudaDev);
  c->windows.clear();
  for (Registration* r : c->regs) delete r;
  c->regs.clear();
  symFree(&c->ws, c->cudaDev);
  if (c->local) cudaFree(c->local);
  if (c->status) cudaFreeHost(c->status);
  if (c->scratchEvent) cudaEventDestroy(c->scratchEvent);
  c->boot.close(!abort);
  c->magic = 0;
  delete c;
  if (prevDev >= 0) cudaSetDevice(prevDev);
  return ncclSuccess;
}

namespace {
std::mutex gNotifyMu;
std::vector<ReleaseFn> gNotifiers;
}  // namespace

void addReleaseNotifier(ReleaseFn fn) {
  std::lock_guard<std::mutex> lk(gNotifyMu);
  for (ReleaseFn f : gNotifiers)
    if (f == fn) return;
  gNotifiers.push_back(fn);
}

void notifyRelease(Comm* c, const void* base) {
  std::vector<ReleaseFn> fns;
  {
    std::lock_guard<std::mutex> lk(gNotifyMu);
    fns = gNotifiers;
  }
  for (ReleaseFn f : fns) f(c, base);
}

ncclResult_t commSymAlloc(Comm* c, size_t bytes, void** ptr) {
  std::unique_ptr<Window> w(new Window());
  uint32_t tag;
  {
    std::lock_guard<std::mutex> lk(c->mu);
    tag = c->symTag;
    c->symTag += 2;
  }
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != c->cudaDev) cudaSetDevice(c->cudaDev);
  ncclResult_t r = symAlloc(c->boot, c->cudaDev, bytes, true, tag, &w->seg);
  if (r == ncclSuccess) {
    cudaMemset(w->seg.peer[c->rank], 0, w->seg.size);
    cudaDeviceSynchronize();
    r = c->boot.barrier();
  }
  if (prev != c->cudaDev && prev >= 0) cudaSetDevice(prev);
  BCHECK(r);
  *ptr = w->seg.peer[c->rank];
  std::lock_guard<std::mutex> lk(c->mu);
  w->id = ++c->windowSeq;
  c->windows[(uintptr_t)*ptr] = std::move(w);
  return ncclSuccess;
}

ncclResult_t commSymFree(Comm* c, void* ptr) {
  std::unique_ptr<Window> w;
  {
    std::lock_guard<std::mutex> lk(c->mu);
    auto it = c->windows.find((uintptr_t)ptr);
    if (it == c->windows.end()) BFAIL(ncclInvalidArgument, "%p is not a symmetric allocation of this communicator", ptr);
    w = std::move(it->second);
    c->windows.erase(it);
  }
  notifyRelease(c, ptr);
  cudaDeviceSynchronize();
  BCHECK(c->boot.barrier());
  return symFree(&w->seg, c->cudaDev);
}

// A buffer inside an ncclCommRegister'ed range is exchanged with the peers the first time a
// collective sees it. Every rank reaches this point in the same call because registration is
// required to be symmetric.
ncclResult_t commRegisterLazy(Comm* c, const void* ptr, size_t bytes) {
  Registration* hit = nullptr;
  {
    std::lock_guard<std::mutex> lk(c->mu);
    for (Registration* r : c->regs)
      if (!r->exchanged && !r->failed && (uintptr_t)ptr >= (uintptr_t)r->base && (uintptr_t)ptr + bytes <= (uintptr_t)r->base + r->size) hit = r;
  }
  if (!hit) return ncclSuccess;
  LocalAlloc la;
  if (!localAllocLookup(hit->base, &la) || !la.vmm) {
    hit->failed = true;  // plain cudaMalloc memory: stays on the staged path
    return ncclSuccess;
  }
  {
    std::lock_guard<std::mutex> lk(c->mu);
    if (c->windows.count((uintptr_t)la.ptr)) { hit->exchanged = true; return ncclSuccess; }
  }
  std::unique_ptr<Window> w(new Window());
  uint32_t tag;
  {
    std::lock_guard<std::mutex> lk(c->mu);
    tag = c->symTag;
    c->symTag += 2;
  }
  ncclResult_t r = symAdopt(c->boot, c->cudaDev, la.ptr, la.size, true, tag, &w->seg);
  if (r != ncclSuccess) { hit->failed = true; return r; }
  w->fromRegister = true;
  hit->exchanged = true;
  std::lock_guard<std::mutex> lk(c->mu);
  w->id = ++c->windowSeq;
  c->windows[(uintptr_t)la.ptr] = std::move(w);
  return ncclSuccess;
}

}  // namespace b200
