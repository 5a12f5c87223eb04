// Shared host-side definitions: limits, result plumbing, logging and the flag table.
#pragma once

#include <cuda_runtime_api.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include <string>

#include "b200coll/nccl.h"

namespace b200 {

constexpr int kMaxRanks = 8;     // one NVSwitch domain
constexpr int kMaxCtas = 128;    // flag slots per communicator; also the CTA ceiling of a kernel
constexpr int kCollThreads = 512;
constexpr int kMaxP2pSubs = 16;     // send/recv sub-channels (CTAs) per peer, at most
constexpr int kBulkStages = 4;            // shared-memory ring of the peer-load reduce (six stages measured no faster between 2 GPUs)
constexpr int kBulkStageBytes = 32 << 10;  // per stage: every rank's tile of the same range
constexpr int kBulkSmemBytes = 128 + kBulkStages * kBulkStageBytes;
constexpr int kReduceThreads = 256;  // reducing kernels: fewer threads, more registers for loads in flight

// ---- logging ------------------------------------------------------------------------------
// Levels and subsystem masks follow the NCCL_DEBUG / NCCL_DEBUG_SUBSYS convention; the role of
// the reference's glog-backed ROCP_{TRACE,INFO,WARNING,ERROR} macros
// (rocprofiler-sdk/source/lib/common/logging.cpp:87-127).
enum LogLevel { LOG_NONE = 0, LOG_WARN = 1, LOG_INFO = 2, LOG_TRACE = 3 };
enum LogSubsys : unsigned {
  SUB_INIT = 1, SUB_COLL = 2, SUB_P2P = 4, SUB_MEM = 8, SUB_BOOT = 16, SUB_TOPO = 32,
  SUB_TRACE = 64, SUB_TUNE = 128, SUB_SHMEM = 256, SUB_ALL = ~0u
};
const char* baseName(const char* path);  // file name without directories (messages never carry build paths)
int logLevel();
unsigned logSubsys();
void logMsg(LogLevel lvl, unsigned subsys, const char* file, int line, const char* fmt, ...)
    __attribute__((format(printf, 5, 6)));
void setLastError(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
const char* lastError();

#define BWARN(...) ::b200::logMsg(::b200::LOG_WARN, ::b200::SUB_ALL, __FILE__, __LINE__, __VA_ARGS__)
#define BINFO(sub, ...)                                                                   \
  do {                                                                                    \
    if (::b200::logLevel() >= ::b200::LOG_INFO)                                           \
      ::b200::logMsg(::b200::LOG_INFO, (sub), __FILE__, __LINE__, __VA_ARGS__);           \
  } while (0)
#define BTRACE(sub, ...)                                                                  \
  do {                                                                                    \
    if (::b200::logLevel() >= ::b200::LOG_TRACE)                                          \
      ::b200::logMsg(::b200::LOG_TRACE, (sub), __FILE__, __LINE__, __VA_ARGS__);          \
  } while (0)

#define BCHECK(call)                                 \
  do {                                               \
    ncclResult_t r__ = (call);                       \
    if (r__ != ncclSuccess) return r__;              \
  } while (0)

#define BCUDA(call)                                                                        \
  do {                                                                                     \
    cudaError_t e__ = (call);                                                              \
    if (e__ != cudaSuccess) {                                                              \
      ::b200::setLastError("%s:%d CUDA error '%s' from %s", ::b200::baseName(__FILE__), __LINE__,            \
                           cudaGetErrorString(e__), #call);                                \
      BWARN("CUDA error '%s' from %s", cudaGetErrorString(e__), #call);                    \
      return ncclUnhandledCudaError;                                                       \
    }                                                                                      \
  } while (0)

#define BFAIL(code, ...)                \
  do {                                  \
    ::b200::setLastError(__VA_ARGS__);  \
    BWARN(__VA_ARGS__);                 \
    return (code);                      \
  } while (0)

// ---- flags ---------------------------------------------------------------------------------
// Every environment variable the library reads, parsed once (the counterpart of
// Flag::Refresh in rocr-runtime/runtime/hsa-runtime/core/util/flag.h:78-299). Each knob is
// read as B200COLL_<NAME>, then as NCCL_<NAME> where NCCL has the same knob.
struct Flags {
  int debugLevel = LOG_WARN;
  unsigned debugSubsys = SUB_ALL;
  std::string debugFile;         // DEBUG_FILE: log lines go to this file instead of stdout/stderr (%h host, %p pid)
  int nvlsEnable = 1;            // NVLS_ENABLE: 0 never, 1 when the box supports multicast
  std::string algo;              // ALGO: "", "ll", "p2p", "nvls"
  int minCtas = 0, maxCtas = 0;  // MIN_CTAS / MAX_CTAS (0: per-collective default)
  size_t stageBytes = 64ull << 20;   // BUFFSIZE: bytes per staging half
  size_t llMaxBytes = 2ull << 20;    // LL_THRESHOLD: largest message for the flag-in-data protocol (see llLimit)
  // Every rank stores its whole message (with as many bytes of flags) into every peer, 2 x bytes x (n - 1) in all, at
  // about 600 GB/s behind a latency of about 8 us; NCCL answers small messages in 20 - 28 us. So the protocol pays up to
  // roughly 4 MiB / (n - 1): 2 MiB between two or three ranks (measured between two: staged 24 - 27 us at 512 KiB - 2 MiB
  // against 19 us for NCCL and 9 - 17 us for this protocol), 1 MiB between four, 512 KiB from five to eight.
  size_t llLimit(int nranks) const {
    const size_t byRanks = nranks <= 3 ? (2ull << 20) : nranks == 4 ? (1ull << 20) : (512ull << 10);
    return llMaxBytes < byRanks ? llMaxBytes : byRanks;
  }
  // Reduce-scatter, all-gather and all-to-all move one slice per peer, 2 x slice x (n - 1) per rank: the limit on a slice
  // (it must also fit a slot of the line buffer, which holds 2 x llLimit bytes of lines).
  size_t llSliceLimit(int nranks) const {
    const size_t whole = llLimit(nranks);
    if (nranks <= 2) return whole;
    const size_t bySlices = whole * 4 / (size_t)nranks;
    return bySlices < whole ? bySlices : whole;
  }
  size_t p2pChunkBytes = 512ull << 10; // P2P_CHUNK: bytes per send/recv FIFO slot
  long long a2aStagedMin = -1;         // A2A_STAGED_MIN: all-to-all chunks (bytes per pair) from this size go through the staging halves; -1: built-in choice (1 MiB)
  int p2pCtasPerPeer = 0;        // P2P_CTAS: CTAs per (peer, direction); 0 picks by rank count
  int waitTimeoutMs = 20000;     // WAIT_TIMEOUT_MS: device-side wait budget
  int bootTimeoutMs = 120000;    // BOOTSTRAP_TIMEOUT_MS: host rendezvous budget
  std::string commId;            // COMM_ID: "ip:port" of the rendezvous root
  std::string ifaddr = "127.0.0.1";  // SOCKET_ADDR: address the root listens on
  std::string tuningFile;        // TUNING_FILE: JSON size->algorithm table
  std::string toolLibs;          // TOOL_LIBRARIES: ':'-separated tools given the dispatch table
  long long pipeChunkBytes = -1;  // PIPELINE_CHUNK: staged-reduce pipeline chunk; -1 picks by size, 0 disables
  int dmaGang = 0;                // DMA_GANG: copy engines per copy-engine transfer; 0 picks by size
  int emulateRanks = 0;           // EMULATE_RANKS: several ranks may share one GPU; such communicators only serve b200collEmu*
  int traceEnable = 0;           // TRACE: record per-collective device timestamps
  std::string traceFile;         // TRACE_FILE: CSV written at communicator destroy
  long long traceMaxRecords = 0; // TRACE_MAX_RECORDS: 0 keeps every record; N keeps the first N per communicator and counts the rest
  std::string failKey;           // FAIL_KEY: host-side fault-injection points (tests)
  int ipcLegacy = 0;             // IPC_MODE_LEGACY: cudaIpc handles instead of VMM fds
  int graphRegister = 1;
  int checkSymmetric = 0;         // CHECK_SYMMETRIC: ranks compare (window, offset) of every collective's buffers before choosing the zero-copy path
  static const Flags& get();
  static void refresh();  // re-read the environment (tests)
};
bool failPoint(const char* name);  // true when FAIL_KEY lists `name`
std::string describeSettings();    // JSON array: every knob with its environment names, value, default and meaning

// ---- dtype helpers -------------------------------------------------------------------------
inline size_t dtypeSize(ncclDataType_t t) {
  switch (t) {
    case ncclInt8: case ncclUint8: case ncclFp8E4M3: case ncclFp8E5M2: return 1;
    case ncclFloat16: case ncclBfloat16: return 2;
    case ncclInt32: case ncclUint32: case ncclFloat32: return 4;
    case ncclInt64: case ncclUint64: case ncclFloat64: return 8;
    default: return 0;
  }
}
const char* dtypeName(ncclDataType_t t);
const char* opName(int op);

uint64_t nowNs();  // CLOCK_MONOTONIC

}  // namespace b200
