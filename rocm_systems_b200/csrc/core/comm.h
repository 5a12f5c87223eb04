// The communicator: bootstrap connection, symmetric workspace, device-visible state, windows
// registered by the user, async error state and the watchdog that feeds it.
//
// Lifetime mirrors the ref-counted runtime singleton of the reference
// (rocr-runtime/runtime/hsa-runtime/core/runtime/runtime.cpp:111-156) at communicator scope:
// ncclCommInitRank* builds one, ncclCommFinalize quiesces it, ncclCommDestroy/Abort free it.
#pragma once

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "../coll/device.h"
#include "bootstrap.h"
#include "common.h"
#include "mem.h"

namespace b200 {

class Tracer;

struct Window {          // a symmetric range usable for zero-copy collectives
  SymSeg seg;
  void* userHandle = nullptr;  // what ncclCommRegister returned, if it came from there
  bool fromRegister = false;
  uint64_t id = 0;             // position in the communicator's sequence of collective window creations: the same on every rank
};

struct Registration {    // ncclCommRegister bookkeeping (local until first collective use)
  void* base;
  size_t size;
  bool exchanged = false;
  bool failed = false;
};

struct PreMulOp {
  bool used = false;
  ncclDataType_t dtype;
  unsigned long long bits;        // host-immediate scalar, in the element type
  const void* devPtr = nullptr;   // device-resident scalar: handed to the kernel, which reads it in stream order
};

struct TuneEntry {       // one row of the size -> algorithm table
  int coll;              // CollKind, or -1 for any
  size_t maxBytes;       // applies to messages up to this many bytes
  int algo;              // Algo
  int ctas;
};
enum Algo : int { ALGO_AUTO = 0, ALGO_LL = 1, ALGO_P2P = 2, ALGO_NVLS = 3 };

// The ranks of one communicator that live in this process (ncclCommInitAll, or one thread per rank). Tearing a
// communicator down is collective (every rank must have finished its device work before anyone unbinds memory), so a
// thread that destroys its ranks one after the other would wait for ranks it has not come to yet: their teardown is
// deferred until the last of them has been asked for and then runs for all of them at once.
struct Comm;
struct LocalGroup {
  std::mutex mu;
  int members = 0;
  std::vector<Comm*> waiting;
};

struct Comm {
  uint64_t magic = 0;
  int rank = -1, nranks = 0, cudaDev = -1;
  ncclConfig_t config{};
  Bootstrap boot;
  SymSeg ws;                         // workspace
  DevComm dev{};                     // template of what every kernel launch receives
  LocalState* local = nullptr;       // device memory
  DevStatus* status = nullptr;       // mapped host memory
  uint32_t* abortFlag = nullptr;     // mapped host memory
  bool nvls = false;                 // workspace has a multicast alias
  bool emulated = false;             // shares its GPU with other ranks of the communicator: only b200collEmu* may launch on it
  uint64_t opSeq = 0;
  uint32_t llSeq = 0;
  uint32_t stageParity = 0;
  uint32_t symTag = 100;             // next tag for descriptor exchanges
  int maxCtas = 32, minCtas = 1;
  std::mutex mu;
  std::map<uintptr_t, std::unique_ptr<Window>> windows;   // keyed by local base address
  uint64_t windowSeq = 0;                                  // windows created so far (creation is collective)
  std::vector<Registration*> regs;
  std::vector<PreMulOp> premul;
  std::vector<TuneEntry> tuning;
  std::atomic<int> asyncError{ncclSuccess};
  std::atomic<bool> finalized{false}, aborted{false}, destroyRequested{false};
  std::shared_ptr<LocalGroup> localGroup;
  std::string lastErr;
  std::thread watchdog;
  std::atomic<bool> stopWatchdog{false};
  Tracer* tracer = nullptr;
  cudaEvent_t scratchEvent = nullptr;

  // Finds the window containing [ptr, ptr+bytes) and the offset of ptr inside it.
  Window* findWindow(const void* ptr, size_t bytes, size_t* off);
};
extern thread_local bool tlsEmuCall;  // set while a b200collEmu* entry point runs on this thread
constexpr uint64_t kCommMagic = 0xb200c0440000c033ull;

ncclResult_t commCreate(Comm** out, const ncclUniqueId& id, int nranks, int rank, const ncclConfig_t* config);
ncclResult_t commDestroy(Comm* c, bool abort);
ncclResult_t commCheck(const Comm* c);                 // valid and not in error
ncclResult_t commPollStatus(Comm* c);                  // fold the device status word into asyncError
ncclResult_t commRegisterLazy(Comm* c, const void* ptr, size_t bytes);  // exchange a registration on first use
ncclResult_t commSymAlloc(Comm* c, size_t bytes, void** ptr);
ncclResult_t commSymFree(Comm* c, void* ptr);
// Release notifiers (the allocation-map notifiers of an HSA runtime, rocr-runtime core/runtime/runtime.cpp:313-467, for
// symmetric memory): code that keeps host state per (communicator, symmetric allocation) registers a function that runs
// when the allocation is freed (base = its address) and when the communicator goes away (base = nullptr), so that a
// later allocation at the same address starts from a clean slate. Registering a function twice keeps one entry.
using ReleaseFn = void (*)(Comm* c, const void* base);
void addReleaseNotifier(ReleaseFn fn);
void notifyRelease(Comm* c, const void* base);
void loadTuning(Comm* c);

inline Comm* asComm(ncclComm_t c) { return const_cast<Comm*>(reinterpret_cast<const Comm*>(c)); }

}  // namespace b200
