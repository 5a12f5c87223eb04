#include "common.h"

#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#include <mutex>

namespace b200 {

static std::mutex gFlagMu;
static Flags* gFlags = nullptr;

static const char* envOf(const char* name, bool ncclToo = true) {
  std::string a = std::string("B200COLL_") + name;
  const char* v = getenv(a.c_str());
  if (v && *v) return v;
  if (ncclToo) {
    std::string b = std::string("NCCL_") + name;
    v = getenv(b.c_str());
    if (v && *v) return v;
  }
  return nullptr;
}

static size_t parseSize(const char* s, size_t dflt) {
  if (!s) return dflt;
  char* end = nullptr;
  double v = strtod(s, &end);
  if (end == s) return dflt;
  switch (*end) {
    case 'k': case 'K': v *= 1024.0; break;
    case 'm': case 'M': v *= 1024.0 * 1024.0; break;
    case 'g': case 'G': v *= 1024.0 * 1024.0 * 1024.0; break;
    default: break;
  }
  return (size_t)v;
}

static int parseInt(const char* s, int dflt) { return s ? atoi(s) : dflt; }

static unsigned parseSubsys(const char* s) {
  if (!s) return SUB_ALL;
  unsigned m = 0;
  std::string str(s);
  size_t pos = 0;
  while (pos <= str.size()) {
    size_t c = str.find(',', pos);
    std::string tok = str.substr(pos, c == std::string::npos ? std::string::npos : c - pos);
    for (auto& ch : tok) ch = toupper(ch);
    if (tok == "INIT") m |= SUB_INIT;
    else if (tok == "COLL") m |= SUB_COLL;
    else if (tok == "P2P") m |= SUB_P2P;
    else if (tok == "MEM" || tok == "ALLOC") m |= SUB_MEM;
    else if (tok == "BOOTSTRAP" || tok == "NET") m |= SUB_BOOT;
    else if (tok == "GRAPH" || tok == "TOPO") m |= SUB_TOPO;
    else if (tok == "TRACE" || tok == "PROFILE") m |= SUB_TRACE;
    else if (tok == "TUNING") m |= SUB_TUNE;
    else if (tok == "SHMEM") m |= SUB_SHMEM;
    else if (tok == "ALL") m = SUB_ALL;
    if (c == std::string::npos) break;
    pos = c + 1;
  }
  return m ? m : SUB_ALL;
}

static void load(Flags& f) {
  if (const char* v = envOf("DEBUG")) {
    std::string s(v);
    for (auto& ch : s) ch = toupper(ch);
    if (s == "WARN") f.debugLevel = LOG_WARN;
    else if (s == "INFO") f.debugLevel = LOG_INFO;
    else if (s == "TRACE") f.debugLevel = LOG_TRACE;
    else if (s == "NONE" || s == "VERSION") f.debugLevel = LOG_NONE;
  }
  f.debugSubsys = parseSubsys(envOf("DEBUG_SUBSYS"));
  f.nvlsEnable = parseInt(envOf("NVLS_ENABLE"), f.nvlsEnable);
  if (const char* v = envOf("ALGO")) {
    f.algo = v;
    for (auto& ch : f.algo) ch = tolower(ch);
  }
  f.minCtas = parseInt(envOf("MIN_CTAS"), 0);
  f.maxCtas = parseInt(envOf("MAX_CTAS"), 0);
  f.stageBytes = parseSize(envOf("BUFFSIZE"), f.stageBytes);
  f.llMaxBytes = parseSize(envOf("LL_THRESHOLD", false), f.llMaxBytes);
  f.p2pChunkBytes = parseSize(envOf("P2P_CHUNK", false), f.p2pChunkBytes);
  f.p2pCtasPerPeer = parseInt(envOf("P2P_CTAS", false), f.p2pCtasPerPeer);
  if (const char* v = envOf("PIPELINE_CHUNK", false)) f.pipeChunkBytes = (long long)parseSize(v, 0);
  f.waitTimeoutMs = parseInt(envOf("WAIT_TIMEOUT_MS", false), f.waitTimeoutMs);
  f.bootTimeoutMs = parseInt(envOf("BOOTSTRAP_TIMEOUT_MS", false), f.bootTimeoutMs);
  if (const char* v = envOf("COMM_ID")) f.commId = v;
  if (const char* v = envOf("SOCKET_ADDR", false)) f.ifaddr = v;
  if (const char* v = envOf("TUNING_FILE", false)) f.tuningFile = v;
  if (const char* v = envOf("TOOL_LIBRARIES", false)) f.toolLibs = v;
  f.traceEnable = parseInt(envOf("TRACE", false), 0);
  if (const char* v = envOf("TRACE_FILE", false)) f.traceFile = v;
  if (const char* v = envOf("FAIL_KEY", false)) f.failKey = v;
  f.ipcLegacy = parseInt(envOf("IPC_MODE_LEGACY", false), 0);
  // Sanity clamps: sizes must stay multiples of what the kernels vectorise on.
  if (f.stageBytes < (1u << 20)) f.stageBytes = 1u << 20;
  f.stageBytes &= ~(size_t)0xffff;
  if (f.llMaxBytes > (256u << 10)) f.llMaxBytes = 256u << 10;
  f.llMaxBytes &= ~(size_t)0xff;
  if (f.p2pChunkBytes < (64u << 10)) f.p2pChunkBytes = 64u << 10;
  f.p2pChunkBytes &= ~(size_t)0xfff;
  if (f.p2pCtasPerPeer < 0) f.p2pCtasPerPeer = 0;
  if (f.p2pCtasPerPeer > kMaxP2pSubs) f.p2pCtasPerPeer = kMaxP2pSubs;
  if (f.waitTimeoutMs < 1) f.waitTimeoutMs = 1;
}

const Flags& Flags::get() {
  std::lock_guard<std::mutex> lk(gFlagMu);
  if (!gFlags) {
    gFlags = new Flags();
    load(*gFlags);
  }
  return *gFlags;
}

void Flags::refresh() {
  std::lock_guard<std::mutex> lk(gFlagMu);
  Flags* f = new Flags();
  load(*f);
  gFlags = f;  // the old table is leaked on purpose: readers may still hold a reference
}

bool failPoint(const char* name) {
  const std::string& k = Flags::get().failKey;
  if (k.empty()) return false;
  size_t pos = 0;
  std::string n(name);
  while (pos <= k.size()) {
    size_t c = k.find(',', pos);
    std::string tok = k.substr(pos, c == std::string::npos ? std::string::npos : c - pos);
    if (tok == n) return true;
    if (c == std::string::npos) break;
    pos = c + 1;
  }
  return false;
}

int logLevel() { return Flags::get().debugLevel; }
unsigned logSubsys() { return Flags::get().debugSubsys; }

void logMsg(LogLevel lvl, unsigned subsys, const char* file, int line, const char* fmt, ...) {
  if (lvl > logLevel()) return;
  if (lvl > LOG_WARN && !(subsys & logSubsys())) return;
  char buf[1024];
  const char* base = strrchr(file, '/');
  base = base ? base + 1 : file;
  char host[64] = "";
  gethostname(host, sizeof(host) - 1);
  int n = snprintf(buf, sizeof(buf), "%s:%d b200coll %s %s:%d ", host, (int)getpid(),
                   lvl == LOG_WARN ? "WARN" : (lvl == LOG_INFO ? "INFO" : "TRACE"), base, line);
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf + n, sizeof(buf) - n, fmt, ap);
  va_end(ap);
  fprintf(lvl == LOG_WARN ? stderr : stdout, "%s\n", buf);
  fflush(lvl == LOG_WARN ? stderr : stdout);
}

static thread_local char tlsLastError[1024] = "";
static char gLastError[1024] = "";
static std::mutex gErrMu;

void setLastError(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tlsLastError, sizeof(tlsLastError), fmt, ap);
  va_end(ap);
  std::lock_guard<std::mutex> lk(gErrMu);
  memcpy(gLastError, tlsLastError, sizeof(gLastError));
}

const char* lastError() { return tlsLastError[0] ? tlsLastError : gLastError; }

const char* dtypeName(ncclDataType_t t) {
  static const char* names[] = {"int8", "uint8", "int32", "uint32", "int64", "uint64", "half",
                                "float", "double", "bfloat16", "fp8_e4m3", "fp8_e5m2"};
  return (int)t >= 0 && (int)t < ncclNumTypes ? names[t] : "?";
}

const char* opName(int op) {
  static const char* names[] = {"sum", "prod", "max", "min", "avg"};
  if (op >= 0 && op < ncclNumOps) return names[op];
  return "mulsum";
}

uint64_t nowNs() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + ts.tv_nsec;
}

}  // namespace b200
