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
  if (const char* v = envOf("DEBUG_FILE")) {
    // %h -> host name, %p -> process id, so every rank can write its own file
    char host[64] = "";
    gethostname(host, sizeof(host) - 1);
    for (const char* c = v; *c; ++c) {
      if (c[0] == '%' && c[1] == 'h') { f.debugFile += host; ++c; }
      else if (c[0] == '%' && c[1] == 'p') { f.debugFile += std::to_string((long)getpid()); ++c; }
      else f.debugFile += *c;
    }
  }
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
  if (const char* v = envOf("A2A_STAGED_MIN", false)) f.a2aStagedMin = (long long)parseSize(v, 0);
  f.p2pCtasPerPeer = parseInt(envOf("P2P_CTAS", false), f.p2pCtasPerPeer);
  if (const char* v = envOf("PIPELINE_CHUNK", false)) f.pipeChunkBytes = (long long)parseSize(v, 0);
  f.dmaGang = parseInt(envOf("DMA_GANG", false), f.dmaGang);
  f.emulateRanks = parseInt(envOf("EMULATE_RANKS", false), f.emulateRanks);
  f.waitTimeoutMs = parseInt(envOf("WAIT_TIMEOUT_MS", false), f.waitTimeoutMs);
  f.bootTimeoutMs = parseInt(envOf("BOOTSTRAP_TIMEOUT_MS", false), f.bootTimeoutMs);
  if (const char* v = envOf("COMM_ID")) f.commId = v;
  if (const char* v = envOf("SOCKET_ADDR", false)) f.ifaddr = v;
  if (const char* v = envOf("TUNING_FILE", false)) f.tuningFile = v;
  if (const char* v = envOf("TOOL_LIBRARIES", false)) f.toolLibs = v;
  f.traceEnable = parseInt(envOf("TRACE", false), 0);
  if (const char* v = envOf("TRACE_FILE", false)) f.traceFile = v;
  f.traceMaxRecords = parseInt(envOf("TRACE_MAX_RECORDS", false), 0);
  if (f.traceMaxRecords < 0) f.traceMaxRecords = 0;
  if (const char* v = envOf("FAIL_KEY", false)) f.failKey = v;
  f.ipcLegacy = parseInt(envOf("IPC_MODE_LEGACY", false), 0);
  f.checkSymmetric = parseInt(envOf("CHECK_SYMMETRIC", false), 0);
  // Sanity clamps: sizes must stay multiples of what the kernels vectorise on.
  if (f.stageBytes < (1u << 20)) f.stageBytes = 1u << 20;
  f.stageBytes &= ~(size_t)0xffff;
  if (f.llMaxBytes > (2u << 20)) f.llMaxBytes = 2u << 20;
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

const char* baseName(const char* path) {
  const char* b = strrchr(path, '/');
  return b ? b + 1 : path;
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
  FILE* out = lvl == LOG_WARN ? stderr : stdout;
  const std::string& path = Flags::get().debugFile;
  if (!path.empty()) {
    static std::mutex fileMu;
    static FILE* logFile = nullptr;
    static std::string opened;
    std::lock_guard<std::mutex> lk(fileMu);
    if (!logFile || opened != path) {  // the path can change when tests re-read the environment
      if (logFile) fclose(logFile);
      logFile = fopen(path.c_str(), "a");
      opened = path;
    }
    if (logFile) out = logFile;
    fprintf(out, "%s\n", buf);
    fflush(out);
    return;
  }
  fprintf(out, "%s\n", buf);
  fflush(out);
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

namespace b200 {
// ---- settings listing --------------------------------------------------------------------------
// Every knob with its environment names, current value, default and meaning, as JSON: what
// `python -m rocm_systems_b200.tools.avail` prints (the role rocprof-sys-avail plays for its
// settings: rocprofiler-systems/source/bin/rocprof-sys-avail).
namespace {
struct SettingDoc {
  const char* name;
  bool ncclAlias;
  const char* dflt;
  const char* doc;
};
const SettingDoc kSettings[] = {
    {"DEBUG", true, "WARN", "log level: NONE, WARN, INFO, TRACE"},
    {"DEBUG_FILE", true, "", "write log lines to this file instead of stdout / stderr; %h is the host name, %p the process id"},
    {"DEBUG_SUBSYS", true, "ALL", "comma list of INIT,COLL,P2P,MEM,BOOTSTRAP,TOPO,TRACE,TUNING,SHMEM for INFO/TRACE lines"},
    {"NVLS_ENABLE", true, "1", "0: never use in-switch reduction / multicast; 1: when the box supports it"},
    {"ALGO", true, "", "force an algorithm: ll, p2p or nvls (a forced choice that cannot serve a call falls back)"},
    {"MIN_CTAS", true, "0", "lower bound of CTAs per collective launch (0: built-in)"},
    {"MAX_CTAS", true, "0", "upper bound of CTAs per collective launch (0: built-in)"},
    {"BUFFSIZE", true, "64M", "bytes per staging half (two halves per communicator), at least 1M"},
    {"LL_THRESHOLD", false, "2M", "largest all-reduce served by the flag-in-data protocol: at most 2M up to three ranks, 1M between four, 512K from five to eight"},
    {"P2P_CHUNK", false, "512K", "bytes per send/recv FIFO slot"},
    {"A2A_STAGED_MIN", false, "-1", "all-to-all: chunks (bytes per pair) from this size move through the staging halves by peer stores instead of the send/recv FIFOs (-1: built-in choice, 1 MiB)"},
    {"P2P_CTAS", false, "0", "CTAs per peer and direction for send/recv (0: 16 / 8 / 4 for 2 / up to 4 / more ranks)"},
    {"PIPELINE_CHUNK", false, "-1", "pipeline chunk of the staged reductions in bytes (-1: by message size, 0: no chunking)"},
    {"DMA_GANG", false, "0", "copy engines one copy-engine put/get is split over (0: 1, 2 or 4 by size; at most 8)"},
    {"CHECK_SYMMETRIC", false, "0", "1: before a collective takes the zero-copy path the ranks compare, over the rendezvous network, which window and offset "
                                   "each of them passed; on any difference all of them stage instead (a host exchange per call: for debugging)"},
    {"EMULATE_RANKS", false, "0", "1: ranks may share a GPU; their communicators serve only the b200collEmu* entry points, which play all ranks in one kernel (tests)"},
    {"WAIT_TIMEOUT_MS", false, "20000", "budget of every device-side wait; on expiry the kernel records the wait and returns"},
    {"BOOTSTRAP_TIMEOUT_MS", false, "120000", "budget of the host rendezvous"},
    {"COMM_ID", true, "", "ip:port of the rendezvous root (ncclGetUniqueId then needs no out-of-band exchange)"},
    {"SOCKET_ADDR", false, "127.0.0.1", "address the rendezvous root listens on"},
    {"TUNING_FILE", false, "", "JSON table of rows {coll, max_bytes, algo, ctas} consulted before the built-in thresholds"},
    {"TOOL_LIBRARIES", false, "", "':'-separated shared objects given the dispatch table through b200coll_tool_configure"},
    {"TRACE", false, "0", "1: record host and device times of every collective (and b200tx ranges)"},
    {"TRACE_FILE", false, "", "prefix of the CSV files written when a communicator is destroyed / at exit"},
    {"TRACE_MAX_RECORDS", false, "0", "0: keep every collective record (lossless); N: keep the first N per communicator, count the rest as dropped"},
    {"FAIL_KEY", false, "", "comma list of host-side fault-injection points (tests only)"},
    {"IPC_MODE_LEGACY", false, "0", "1: share memory through cudaIpc handles instead of VMM file descriptors"},
};

std::string currentValue(const Flags& f, const std::string& n) {
  auto num = [](long long v) { return std::to_string(v); };
  if (n == "DEBUG") return f.debugLevel == LOG_NONE ? "NONE" : f.debugLevel == LOG_WARN ? "WARN" : f.debugLevel == LOG_INFO ? "INFO" : "TRACE";
  if (n == "DEBUG_FILE") return f.debugFile;
  if (n == "DEBUG_SUBSYS") return f.debugSubsys == SUB_ALL ? "ALL" : num(f.debugSubsys);
  if (n == "NVLS_ENABLE") return num(f.nvlsEnable);
  if (n == "ALGO") return f.algo;
  if (n == "MIN_CTAS") return num(f.minCtas);
  if (n == "MAX_CTAS") return num(f.maxCtas);
  if (n == "BUFFSIZE") return num((long long)f.stageBytes);
  if (n == "LL_THRESHOLD") return num((long long)f.llMaxBytes);
  if (n == "P2P_CHUNK") return num((long long)f.p2pChunkBytes);
  if (n == "A2A_STAGED_MIN") return num(f.a2aStagedMin);
  if (n == "P2P_CTAS") return num(f.p2pCtasPerPeer);
  if (n == "PIPELINE_CHUNK") return num(f.pipeChunkBytes);
  if (n == "DMA_GANG") return num(f.dmaGang);
  if (n == "EMULATE_RANKS") return num(f.emulateRanks);
  if (n == "CHECK_SYMMETRIC") return num(f.checkSymmetric);
  if (n == "WAIT_TIMEOUT_MS") return num(f.waitTimeoutMs);
  if (n == "BOOTSTRAP_TIMEOUT_MS") return num(f.bootTimeoutMs);
  if (n == "COMM_ID") return f.commId;
  if (n == "SOCKET_ADDR") return f.ifaddr;
  if (n == "TUNING_FILE") return f.tuningFile;
  if (n == "TOOL_LIBRARIES") return f.toolLibs;
  if (n == "TRACE") return num(f.traceEnable);
  if (n == "TRACE_FILE") return f.traceFile;
  if (n == "TRACE_MAX_RECORDS") return num(f.traceMaxRecords);
  if (n == "FAIL_KEY") return f.failKey;
  if (n == "IPC_MODE_LEGACY") return num(f.ipcLegacy);
  return "";
}

std::string jsonEscape(const std::string& s) {
  std::string o;
  for (char ch : s) {
    if (ch == '"' || ch == '\\') o += '\\';
    if ((unsigned char)ch < 0x20) continue;
    o += ch;
  }
  return o;
}
}  // namespace

std::string describeSettings() {
  const Flags& f = Flags::get();
  std::string out = "[";
  bool first = true;
  for (const SettingDoc& s : kSettings) {
    if (!first) out += ",";
    first = false;
    out += std::string("{\"name\":\"") + s.name + "\",\"env\":[\"B200COLL_" + s.name + "\"" + (s.ncclAlias ? std::string(",\"NCCL_") + s.name + "\"" : "") +
           "],\"value\":\"" + jsonEscape(currentValue(f, s.name)) + "\",\"default\":\"" + s.dflt + "\",\"doc\":\"" + jsonEscape(s.doc) + "\"}";
  }
  return out + "]";
}
}  // namespace b200
