#include "b200coll/markers.h"

#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <limits.h>
#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../core/common.h"

namespace {

std::mutex gMu;
std::vector<b200tx_record_t> gDone;
std::map<uint64_t, b200tx_record_t> gOpen;   // started with RangeStart
std::atomic<uint64_t> gNextId{1};
std::atomic<int> gEnabled{-1};                // -1: not decided yet
thread_local std::vector<b200tx_record_t> tlsStack;

// With B200COLL_TRACE=1 and B200COLL_TRACE_FILE=<prefix> the finished ranges of the process are
// written to <prefix>.markers.<pid>.csv when it exits.
void writeAtExit() {
  const std::string& prefix = b200::Flags::get().traceFile;
  if (prefix.empty()) return;
  std::lock_guard<std::mutex> lk(gMu);
  if (gDone.empty()) return;
  char path[512];
  snprintf(path, sizeof(path), "%s.markers.%d.csv", prefix.c_str(), (int)getpid());
  FILE* f = fopen(path, "w");
  if (!f) return;
  fprintf(f, "\"Domain\",\"Function\",\"Process_Id\",\"Thread_Id\",\"Correlation_Id\",\"Start_Timestamp\",\"End_Timestamp\",\"Depth\"\n");
  for (const auto& r : gDone) {
    char msg[sizeof(r.message)];
    memcpy(msg, r.message, sizeof(msg));
    for (char* c = msg; *c; ++c)
      if (*c == '"') *c = '\'';
    fprintf(f, "\"MARKER_API\",\"%s\",%d,%u,%llu,%llu,%llu,%u\n", msg, (int)getpid(), r.tid, (unsigned long long)r.id,
            (unsigned long long)r.beginNs, (unsigned long long)r.endNs, r.depth);
  }
  fclose(f);
}

// A traced program that is ended by a signal would leave no file: with B200COLL_TRACE_SIGNALS=1 (the tracing launcher sets
// it unless told otherwise) the ranges are written when SIGTERM, SIGINT, SIGQUIT or SIGABRT arrives, then the signal takes
// its default course. Only where the program has no handler of its own for that signal. The reference's launcher installs
// the same kind of handlers (rocprofv3 --disable-signal-handlers switches them off) so that an aborted run keeps its output.
void onFatalSignal(int sig) {
  static std::atomic<int> once{0};
  if (once.exchange(1) == 0) {
    if (gMu.try_lock()) {  // the interrupted thread may hold it: then there is nothing safe to do
      gMu.unlock();
      writeAtExit();
    }
  }
  signal(sig, SIG_DFL);
  raise(sig);
}

void installSignalFlush() {
  const char* v = getenv("B200COLL_TRACE_SIGNALS");
  if (!v || !*v || !strcmp(v, "0")) return;
  for (int sig : {SIGTERM, SIGINT, SIGQUIT, SIGABRT}) {
    struct sigaction old;
    if (sigaction(sig, nullptr, &old) != 0 || old.sa_handler != SIG_DFL) continue;
    struct sigaction sa;
    memset(&sa, 0, sizeof(sa));
    sa.sa_handler = onFatalSignal;
    sigemptyset(&sa.sa_mask);
    sigaction(sig, &sa, nullptr);
  }
}

bool enabled() {
  int e = gEnabled.load();
  if (e < 0) {
    e = b200::Flags::get().traceEnable ? 1 : 0;
    int expected = -1;
    if (gEnabled.compare_exchange_strong(expected, e) && e == 1) {
      atexit(writeAtExit);
      installSignalFlush();
    }
  }
  return gEnabled.load() == 1;
}

b200tx_record_t make(const char* msg, uint64_t id, uint32_t depth) {
  b200tx_record_t r{};
  r.id = id;
  r.beginNs = r.endNs = b200::nowNs();
  r.tid = (uint32_t)syscall(SYS_gettid);
  r.depth = depth;
  if (msg) strncpy(r.message, msg, sizeof(r.message) - 1);
  return r;
}

}  // namespace

extern "C" {

void b200txEnable(int on) { gEnabled.store(on ? 1 : 0); }

void b200txMark(const char* message) {
  if (!enabled()) return;
  b200tx_record_t r = make(message, 0, (uint32_t)tlsStack.size());
  std::lock_guard<std::mutex> lk(gMu);
  gDone.push_back(r);
}

int b200txRangePush(const char* message) {
  if (!enabled()) return -1;
  tlsStack.push_back(make(message, gNextId.fetch_add(1), (uint32_t)tlsStack.size()));
  return (int)tlsStack.size() - 1;
}

int b200txRangePop(void) {
  if (tlsStack.empty()) return -1;
  b200tx_record_t r = tlsStack.back();
  tlsStack.pop_back();
  r.endNs = b200::nowNs();
  std::lock_guard<std::mutex> lk(gMu);
  gDone.push_back(r);
  return (int)r.depth;
}

uint64_t b200txRangeStart(const char* message) {
  if (!enabled()) return 0;
  b200tx_record_t r = make(message, gNextId.fetch_add(1), 0);
  std::lock_guard<std::mutex> lk(gMu);
  gOpen[r.id] = r;
  return r.id;
}

void b200txRangeStop(uint64_t id) {
  std::lock_guard<std::mutex> lk(gMu);
  auto it = gOpen.find(id);
  if (it == gOpen.end()) return;
  it->second.endNs = b200::nowNs();
  gDone.push_back(it->second);
  gOpen.erase(it);
}

uint64_t b200txRangeAt(const char* message, uint64_t beginNs, uint64_t endNs) {
  if (!enabled()) return 0;
  b200tx_record_t r = make(message, gNextId.fetch_add(1), (uint32_t)tlsStack.size());
  r.beginNs = beginNs;
  r.endNs = endNs < beginNs ? beginNs : endNs;
  std::lock_guard<std::mutex> lk(gMu);
  gDone.push_back(r);
  return r.id;
}

uint64_t b200txGet(b200tx_record_t* out, uint64_t max) {
  std::lock_guard<std::mutex> lk(gMu);
  const uint64_t n = gDone.size() < max ? gDone.size() : max;
  if (out && n) memcpy(out, gDone.data(), n * sizeof(b200tx_record_t));
  return gDone.size();
}

void b200txClear(void) {
  std::lock_guard<std::mutex> lk(gMu);
  gDone.clear();
}

const char* b200collBuildInfo(void) {
  static char buf[256];
  int rt = 0;
  cudaRuntimeGetVersion(&rt);
  snprintf(buf, sizeof(buf), "b200coll 0.1.0 (NCCL API %d.%d.%d) sm_100a cuda-runtime %d.%d built " __DATE__, NCCL_MAJOR, NCCL_MINOR, NCCL_PATCH, rt / 1000,
           (rt % 1000) / 10);
  return buf;
}

// Where this library was loaded from, and the directory above its lib/ (the install prefix), found from the address of this
// very function: what the reference's rocm-core answers with getROCmInstallPath (rocm-core/rocm_getpath.cpp).
int b200collGetInstallPath(char* library, size_t libraryLen, char* prefix, size_t prefixLen) {
  Dl_info info;
  if (!dladdr((void*)&b200collGetInstallPath, &info) || !info.dli_fname) return -1;
  char resolved[4096];
  const char* path = realpath(info.dli_fname, resolved) ? resolved : info.dli_fname;
  if (library && libraryLen) snprintf(library, libraryLen, "%s", path);
  if (prefix && prefixLen) {
    std::string p = path;
    for (int up = 0; up < 2; up++) {  // drop the file name, then the lib directory
      const size_t slash = p.rfind('/');
      p = slash == std::string::npos || slash == 0 ? "/" : p.substr(0, slash);
    }
    snprintf(prefix, prefixLen, "%s", p.c_str());
  }
  return 0;
}

}  // extern "C"
