// b200causal — causal profiling of host code: "how much faster would the program get if THIS function were X % faster".
// The answer cannot be read off a flat profile (a function that burns half the CPU time may sit beside the critical path),
// so it is measured: a function cannot be made faster at will, but every OTHER thread can be made slower by the same
// amount, which leaves the same relative timing. An experiment picks a function and a speed-up s; whenever a CPU-time
// sample of some thread lands in that function (callees included), all other threads owe a pause of s x the CPU time that
// sample stands for. The rate at which the program passes its progress points, with the inserted pauses subtracted from
// the clock, is the rate it would have with the function that much faster.
//
// It plays the part of the reference's causal mode (rocprofiler-systems source/lib/rocprof-sys/library/causal/:
// experiment.cpp runs the experiments, sampling.cpp samples, delay.cpp keeps the global and per-thread pause counts,
// components/blocking_gotcha.cpp and unblocking_gotcha.cpp wrap the pthread calls, components/progress_point.cpp counts;
// settings ROCPROFSYS_CAUSAL_* in source/lib/core/config.cpp:706-812; user macros in
// source/lib/rocprof-sys-user/rocprofiler-systems/causal.h). Function scope by default; for a source-line scope the
// launcher decodes the executable's line table and hands the address ranges of the chosen lines over in a file.
//
// Pauses and dependencies. Each thread keeps how much pause it has served (`local`); the experiment keeps how much is owed
// (`gOwed`). A thread serves the difference when it is sampled and before it does anything that can wake another thread
// (unlock, signal, broadcast, post, barrier, exit), so that a pause is never handed on as a head start. A thread that was
// woken by another thread (lock, condition, join, barrier, semaphore) is credited what became owed while it was blocked:
// the thread that woke it has already served that, or is the one being sped up.
//
// Samples come from per-thread CPU-clock events where the kernel allows them, else from ITIMER_PROF (see "sample sources"
// below); either way the kernel signals a thread in proportion to the CPU time it uses. A sample stands for the CPU time its
// thread used since that thread's previous sample, read from the thread's CPU clock, so whatever the real granularity of the
// source is, the arithmetic stays right.
//
// Ways in: LD_PRELOAD=libb200causal.so with B200CAUSAL_FILE (and _BINARY_SCOPE, _FUNCTION_SCOPE, _FUNCTION_EXCLUDE,
// _FIXED_SPEEDUP, _SOURCE_RANGES, _BACKEND, _FREQ, _EXPERIMENT_SECONDS, _DELAY, _DURATION, _END_TO_END, _FILE_RESET, _RANDOM_SEED, _VERBOSE), or
// b200causalStart / b200causalStop from the program. Output: the text format of the Coz profiler (experiment /
// throughput-point / latency-point lines), which `tools/causal.py` turns into speed-up tables.
#include <cxxabi.h>
#include <dlfcn.h>
#include <elf.h>
#include <execinfo.h>
#include <dirent.h>
#include <fcntl.h>
#include <link.h>
#include <linux/perf_event.h>
#include <pthread.h>
#include <semaphore.h>
#include <signal.h>
#include <sys/ioctl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <sys/time.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <regex>
#include <string>
#include <vector>

#define B200CAUSAL_NO_MACROS
#include "b200coll/causal.h"

extern "C" int __pthread_mutex_lock(pthread_mutex_t*);
extern "C" int __pthread_mutex_unlock(pthread_mutex_t*);

namespace {

// ---------------------------------------------------------------- clocks
int64_t monoNs() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (int64_t)ts.tv_sec * 1000000000ll + ts.tv_nsec;
}
int64_t threadCpuNs() {
  timespec ts;
  clock_gettime(CLOCK_THREAD_CPUTIME_ID, &ts);
  return (int64_t)ts.tv_sec * 1000000000ll + ts.tv_nsec;
}
// Sleeps `ns` (a signal does not cut it short) and returns what was really slept.
int64_t pauseNs(int64_t ns) {
  const int64_t t0 = monoNs();
  timespec want{(time_t)(ns / 1000000000ll), (long)(ns % 1000000000ll)}, left{};
  while (clock_nanosleep(CLOCK_MONOTONIC, 0, &want, &left) == EINTR) want = left;
  return monoNs() - t0;
}

// ---------------------------------------------------------------- functions in scope (read once, before sampling starts)
// One address range that can be selected: a function, or one of the ranges the compiler made of a source line. Ranges of
// the same `entry` are sped up together.
struct Func {
  uintptr_t lo, hi;
  std::string name;
  int entry = -1;
};
std::vector<Func>* gFuncs = nullptr;  // sorted by lo, never changed while the handler can run

std::vector<std::regex> regexList(const char* s) {
  std::vector<std::regex> out;
  std::string cur;
  auto flush = [&] {
    if (!cur.empty()) {
      try {
        out.emplace_back(cur, std::regex::ECMAScript | std::regex::optimize);
      } catch (const std::regex_error&) {
        fprintf(stderr, "[b200causal] not a regular expression: %s\n", cur.c_str());
      }
      cur.clear();
    }
  };
  for (const char* p = s ? s : ""; *p; p++) {
    if (*p == ';' || *p == '\t' || *p == '"' || *p == '\'') flush();
    else cur += *p;
  }
  flush();
  return out;
}
bool matchesAny(const std::vector<std::regex>& res, const std::string& s) {
  for (auto& r : res)
    if (std::regex_search(s, r)) return true;
  return false;
}

std::string demangled(const char* name) {
  int status = 0;
  char* d = abi::__cxa_demangle(name, nullptr, nullptr, &status);
  std::string out = (status == 0 && d) ? d : name;
  free(d);
  return out;
}

// FUNC symbols of one ELF file (.symtab where present, else .dynsym), relocated by `bias`.
void readSymbols(const char* path, uintptr_t bias, std::vector<Func>& out) {
  const int fd = open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) return;
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < (off_t)sizeof(ElfW(Ehdr))) { close(fd); return; }
  void* map = mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (map == MAP_FAILED) return;
  const auto* base = (const unsigned char*)map;
  const auto* eh = (const ElfW(Ehdr)*)base;
  const size_t size = (size_t)st.st_size;
  auto inside = [&](uint64_t off, uint64_t len) { return off <= size && len <= size - off; };
  if (memcmp(eh->e_ident, ELFMAG, SELFMAG) == 0 && eh->e_shentsize == sizeof(ElfW(Shdr)) && inside(eh->e_shoff, (uint64_t)eh->e_shnum * sizeof(ElfW(Shdr)))) {
    const auto* sh = (const ElfW(Shdr)*)(base + eh->e_shoff);
    const ElfW(Shdr)* tab = nullptr;
    for (int pass = 0; pass < 2 && !tab; pass++)
      for (int i = 0; i < eh->e_shnum; i++)
        if (sh[i].sh_type == (pass == 0 ? SHT_SYMTAB : SHT_DYNSYM) && sh[i].sh_entsize == sizeof(ElfW(Sym))) { tab = &sh[i]; break; }
    if (tab && tab->sh_link < eh->e_shnum && inside(tab->sh_offset, tab->sh_size)) {
      const ElfW(Shdr)& str = sh[tab->sh_link];
      if (inside(str.sh_offset, str.sh_size) && str.sh_size > 0) {
        const auto* syms = (const ElfW(Sym)*)(base + tab->sh_offset);
        const char* names = (const char*)(base + str.sh_offset);
        const size_t n = tab->sh_size / sizeof(ElfW(Sym));
        for (size_t i = 0; i < n; i++) {
          const ElfW(Sym)& s = syms[i];
          if (ELF64_ST_TYPE(s.st_info) != STT_FUNC || s.st_size == 0 || s.st_shndx == SHN_UNDEF || s.st_name >= str.sh_size) continue;
          if (!memchr(names + s.st_name, 0, str.sh_size - s.st_name)) continue;
          out.push_back({bias + s.st_value, bias + s.st_value + s.st_size, demangled(names + s.st_name), -1});
        }
      }
    }
  }
  munmap(map, size);
}

struct ScopeArgs {
  std::vector<std::regex> binary, function, exclude;
  bool mainOnly;
  std::vector<Func> found;
};

int onObject(dl_phdr_info* info, size_t, void* data) {
  auto& a = *(ScopeArgs*)data;
  const bool isMain = !info->dlpi_name || !info->dlpi_name[0];
  char exe[1024];
  std::string path = info->dlpi_name ? info->dlpi_name : "";
  if (isMain) {
    const ssize_t n = readlink("/proc/self/exe", exe, sizeof(exe) - 1);
    if (n <= 0) return 0;
    exe[n] = 0;
    path = exe;
  }
  if (path.empty() || path[0] != '/') return 0;  // the vdso and the like
  const bool in = a.mainOnly ? isMain : matchesAny(a.binary, path);
  if (!in) return 0;
  std::vector<Func> all;
  readSymbols(isMain ? "/proc/self/exe" : path.c_str(), (uintptr_t)info->dlpi_addr, all);
  for (auto& f : all) {
    if (!a.function.empty() && !matchesAny(a.function, f.name)) continue;
    if (matchesAny(a.exclude, f.name)) continue;
    a.found.push_back(std::move(f));
  }
  return 0;
}

int onMainObject(dl_phdr_info* info, size_t, void* data) {
  *(uintptr_t*)data = (uintptr_t)info->dlpi_addr;
  return 1;  // the executable is the first object
}

// Source scope. The line tables are decoded outside (tools/causal.py reads them with readelf); what arrives here is a
// file of lines "<name>\t<lo>-<hi>,<lo>-<hi>,..." with hexadecimal addresses as they stand in the executable's ELF file.
// Entries are numbered from 1 << 20 so that they cannot collide with function indices.
bool readSourceRanges(const char* path, std::vector<Func>& out) {
  FILE* f = fopen(path, "r");
  if (!f) return false;
  uintptr_t bias = 0;
  dl_iterate_phdr(onMainObject, &bias);
  char* line = nullptr;
  size_t cap = 0;
  int entry = 1 << 20;
  while (getline(&line, &cap, f) > 0) {
    char* tab = strchr(line, '\t');
    if (!tab) continue;
    *tab = 0;
    bool any = false;
    for (char* p = tab + 1; *p;) {
      char* end = nullptr;
      const unsigned long long lo = strtoull(p, &end, 16);
      if (end == p || *end != '-') break;
      p = end + 1;
      const unsigned long long hi = strtoull(p, &end, 16);
      if (end == p) break;
      if (hi > lo) {
        out.push_back({bias + (uintptr_t)lo, bias + (uintptr_t)hi, line, entry});
        any = true;
      }
      p = *end == ',' ? end + 1 : end;
      if (*end != ',') break;
    }
    if (any) entry++;
  }
  free(line);
  fclose(f);
  return true;
}

// Index of the function that holds `pc`, or -1. Read-only binary search: safe in the signal handler.
int funcOf(uintptr_t pc) {
  const auto& v = *gFuncs;
  size_t lo = 0, hi = v.size();
  while (lo < hi) {
    const size_t mid = (lo + hi) / 2;
    if (v[mid].lo <= pc) lo = mid + 1;
    else hi = mid;
  }
  if (lo == 0) return -1;
  return pc < v[lo - 1].hi ? (int)(lo - 1) : -1;
}

// ---------------------------------------------------------------- pauses: what is owed and what each thread has served
std::atomic<bool> gActive{false};         // sampling is on: the wrappers below do their bookkeeping
std::atomic<int64_t> gOwed{0};            // ns of pause every thread owes since the start
std::atomic<int64_t> gSamples{0};         // samples in scope since the start
std::atomic<int> gInHandler{0};

struct Thread {
  std::atomic<int> used{0};
  std::atomic<int64_t> local{0};  // ns served (slept, credited, or exempt as the thread that ran the selected function)
  int64_t owedAtBlock = 0;        // gOwed when this thread entered a blocking call
  int64_t lastCpuNs = 0;          // thread CPU clock at its previous sample
  int blocked = 0;                // inside a blocking call: the handler does not pause it (the wake-up credits it instead)
  int keyed = 0;                  // the exit hook is set (never done inside the handler)
  int perfFd = -1;                // perf backend: this thread's CPU-clock event (threads that started under the profiler)
};
constexpr int kMaxThreads = 2048;
Thread gThreads[kMaxThreads];
__thread Thread* tMe __attribute__((tls_model("initial-exec"))) = nullptr;
pthread_key_t gKey;
bool gKeyMade = false;

// A slot for the calling thread, starting level with what is owed now (or with `inherit`, for a thread just created).
Thread* mySlot(int64_t inherit = -1) {
  if (tMe) return tMe;
  for (int i = 0; i < kMaxThreads; i++) {
    int expect = 0;
    if (gThreads[i].used.load(std::memory_order_relaxed) == 0 && gThreads[i].used.compare_exchange_strong(expect, 1)) {
      Thread* t = &gThreads[i];
      t->local.store(inherit >= 0 ? inherit : gOwed.load());
      t->owedAtBlock = 0;
      t->lastCpuNs = threadCpuNs();
      t->blocked = 0;
      t->keyed = 0;
      t->perfFd = -1;
      tMe = t;
      return t;
    }
  }
  return nullptr;  // more threads than slots: this one is neither paused nor credited
}

// ---------------------------------------------------------------- sample sources
// timer  ITIMER_PROF: one process-wide timer on CPU time; the kernel checks it at scheduler ticks, so a sample stands for a
//        whole tick (10 ms on a 100 Hz kernel) whatever rate was asked for.
// perf   one software CPU-clock event per thread (perf_event_open, driven by a high-resolution timer): samples at the rate
//        asked for, so pauses come in much smaller lumps. Each overflow disables its event (a limit of one), signals the
//        thread that owns it, and the handler arms it again: no ring buffer is mapped, nothing is read from the event.
// The reference offers the same two (ROCPROFSYS_CAUSAL_BACKEND = perf | timer | auto, rocprofiler-systems
// source/lib/core/config.cpp:706-716; source/lib/rocprof-sys/library/perf.cpp).
std::atomic<bool> gPerf{false};
int64_t gPerfPeriodNs = 1000000;
constexpr int kMaxEarly = 1024;  // threads that existed before the profiler started: (tid, fd), closed when it stops
int gEarlyFd[kMaxEarly];
int gEarlyCount = 0;

int openCpuClock(pid_t tid) {
  perf_event_attr a;
  memset(&a, 0, sizeof(a));
  a.size = sizeof(a);
  a.type = PERF_TYPE_SOFTWARE;
  a.config = PERF_COUNT_SW_CPU_CLOCK;
  a.sample_period = (uint64_t)gPerfPeriodNs;
  a.disabled = 1;
  a.exclude_kernel = 1;
  a.exclude_hv = 1;
  const int fd = (int)syscall(SYS_perf_event_open, &a, tid, -1, -1, PERF_FLAG_FD_CLOEXEC);
  if (fd < 0) return -1;
  f_owner_ex owner{F_OWNER_TID, tid};
  if (fcntl(fd, F_SETFL, fcntl(fd, F_GETFL) | O_ASYNC) != 0 || fcntl(fd, F_SETSIG, SIGPROF) != 0 || fcntl(fd, F_SETOWN_EX, &owner) != 0 ||
      ioctl(fd, PERF_EVENT_IOC_REFRESH, 1) != 0) {
    close(fd);
    return -1;
  }
  return fd;
}

// An event for every thread that already runs (the calling thread included). False when the first one cannot be opened:
// the kernel or the container does not allow it.
bool openPerfForExistingThreads() {
  DIR* d = opendir("/proc/self/task");
  if (!d) return false;
  bool any = false;
  while (dirent* e = readdir(d)) {
    if (e->d_name[0] < '0' || e->d_name[0] > '9' || gEarlyCount >= kMaxEarly) continue;
    const int fd = openCpuClock((pid_t)atoi(e->d_name));
    if (fd >= 0) {
      gEarlyFd[gEarlyCount++] = fd;
      any = true;
    }
  }
  closedir(d);
  return any;
}

void closePerf() {
  for (int i = 0; i < gEarlyCount; i++) close(gEarlyFd[i]);
  gEarlyCount = 0;
  for (auto& t : gThreads) {
    const int fd = t.perfFd;
    if (fd >= 0 && t.used.load() == 0) {  // slots still in use close their own when their thread ends
      t.perfFd = -1;
      close(fd);
    }
  }
}

// Outside the handler: make sure the slot goes back when the thread ends.
inline Thread* keyed(Thread* t) {
  if (t && !t->keyed && gKeyMade) {
    t->keyed = 1;
    pthread_setspecific(gKey, t);
  }
  return t;
}

void serve(Thread* t) {
  if (!t) return;
  const int64_t need = gOwed.load(std::memory_order_acquire) - t->local.load(std::memory_order_relaxed);
  if (need > 0) t->local.fetch_add(pauseNs(need), std::memory_order_relaxed);
}
// Before anything that may wake another thread.
inline void beforeWake() {
  if (gActive.load(std::memory_order_relaxed)) serve(keyed(mySlot()));
}
inline Thread* beforeBlock() {
  if (!gActive.load(std::memory_order_relaxed)) return nullptr;
  Thread* t = keyed(mySlot());
  if (t) {
    t->owedAtBlock = gOwed.load(std::memory_order_acquire);
    t->blocked = 1;
  }
  return t;
}
inline void afterBlock(Thread* t, bool wokenByThread) {
  if (!t) return;
  t->blocked = 0;
  if (wokenByThread) {
    const int64_t grew = gOwed.load(std::memory_order_acquire) - t->owedAtBlock;
    if (grew > 0) t->local.fetch_add(grew, std::memory_order_relaxed);
  }
}

void onThreadExit(void* p) {
  // No more samples for this thread: a handler that ran after the slot is released would take a new one and leak it.
  sigset_t s;
  sigemptyset(&s);
  sigaddset(&s, SIGPROF);
  pthread_sigmask(SIG_BLOCK, &s, nullptr);
  Thread* t = (Thread*)p;
  if (gActive.load()) serve(t);
  if (t->perfFd >= 0) {
    close(t->perfFd);
    t->perfFd = -1;
  }
  tMe = nullptr;
  t->used.store(0, std::memory_order_release);
}

// ---------------------------------------------------------------- progress points
struct Point {
  std::atomic<const char*> name{nullptr};
  std::atomic<int64_t> visits{0}, begins{0}, ends{0};
};
constexpr int kMaxPoints = 512;
Point gPoints[kMaxPoints];

Point* pointFor(const char* name) {
  if (!name) name = "";
  uint64_t h = 1469598103934665603ull;
  for (const char* p = name; *p; p++) h = (h ^ (unsigned char)*p) * 1099511628211ull;
  for (int probe = 0; probe < kMaxPoints; probe++) {
    Point& pt = gPoints[(h + probe) % kMaxPoints];
    const char* have = pt.name.load(std::memory_order_acquire);
    if (!have) {
      char* copy = strdup(name);
      if (pt.name.compare_exchange_strong(have, copy)) return &pt;
      free(copy);  // another thread took the slot: `have` is its name now
    }
    if (!strcmp(have, name)) return &pt;
  }
  return nullptr;
}

// ---------------------------------------------------------------- the running experiment
struct Experiment {
  std::atomic<bool> running{false};
  std::atomic<int> selected{-1};  // `entry` of the ranges being sped up
  std::atomic<int> percent{0};
  std::atomic<int64_t> selectedSamples{0};
};
Experiment gExp;

constexpr int kRecent = 4096;             // functions of the latest in-scope samples: what the next experiment draws from
std::atomic<int32_t> gRecent[kRecent];
std::atomic<uint64_t> gRecentNext{0};
pid_t gControllerTid = 0;
constexpr int kMaxDepth = 32;

void onSample(int, siginfo_t* info, void*) {
  if (!gActive.load(std::memory_order_relaxed)) return;
  const int saved = errno;
  const int armFd = (info && info->si_code == POLL_HUP && gPerf.load(std::memory_order_relaxed)) ? info->si_fd : -1;
  gInHandler.fetch_add(1, std::memory_order_acquire);
  Thread* me = mySlot();
  if (me && (pid_t)syscall(SYS_gettid) != gControllerTid) {
    const int64_t cpu = threadCpuNs();
    const int64_t stands = cpu - me->lastCpuNs;  // CPU time this sample stands for
    me->lastCpuNs = cpu;
    void* pc[kMaxDepth];
    const int depth = backtrace(pc, kMaxDepth);
    // pc[0] is this handler, pc[1] the signal trampoline, pc[2] the interrupted instruction, the rest return addresses.
    const bool running = gExp.running.load(std::memory_order_acquire);
    const int selected = gExp.selected.load(std::memory_order_relaxed);
    bool hit = false;
    int found[4], nFound = 0;  // the innermost few distinct ranges in scope: callers are candidates too (their time includes the callees')
    for (int i = 2; i < depth; i++) {
      const int r = funcOf((uintptr_t)pc[i] - (i > 2 ? 1 : 0));
      if (r < 0) continue;
      if (nFound < 4 && (nFound == 0 || found[nFound - 1] != r)) found[nFound++] = r;
      if (running && (*gFuncs)[r].entry == selected) hit = true;
      if (nFound == 4 && (hit || !running)) break;
    }
    if (nFound > 0) gSamples.fetch_add(1, std::memory_order_relaxed);
    for (int k = 0; k < nFound; k++) gRecent[gRecentNext.fetch_add(1, std::memory_order_relaxed) % kRecent].store(found[k], std::memory_order_relaxed);
    if (hit) {
      gExp.selectedSamples.fetch_add(1, std::memory_order_relaxed);
      const int64_t owe = stands > 0 ? stands * gExp.percent.load(std::memory_order_relaxed) / 100 : 0;
      if (owe > 0) {
        me->local.fetch_add(owe, std::memory_order_relaxed);  // the thread being sped up does not pause for its own sample
        gOwed.fetch_add(owe, std::memory_order_release);
      }
    }
    if (!me->blocked) {
      serve(me);
      me->lastCpuNs = threadCpuNs();
    }
  }
  if (armFd >= 0) ioctl(armFd, PERF_EVENT_IOC_REFRESH, 1);  // the overflow disabled the event: one more sample, please
  gInHandler.fetch_sub(1, std::memory_order_release);
  errno = saved;
}

// ---------------------------------------------------------------- configuration, output, the experiment loop
struct Config {
  std::string file;
  std::vector<int> speedups;
  double freqHz = 1000.0, experimentSeconds = 0.5, delaySeconds = 0.0, durationSeconds = 0.0;
  bool endToEnd = false, verbose = false;
  uint64_t seed = 0;
  std::string backend = "auto";
};
Config* gCfg = nullptr;
pthread_t gController;
bool gControllerUp = false;
std::atomic<bool> gStopping{false};
std::atomic<uint64_t> gDone{0};
struct sigaction gOldAction;
int64_t gStartNs = 0;

struct Snapshot {
  int64_t ns, owed, visits[kMaxPoints], begins[kMaxPoints], ends[kMaxPoints];
};
void snapshot(Snapshot& s) {
  s.ns = monoNs();
  s.owed = gOwed.load();
  for (int i = 0; i < kMaxPoints; i++) {
    s.visits[i] = gPoints[i].visits.load(std::memory_order_relaxed);
    s.begins[i] = gPoints[i].begins.load(std::memory_order_relaxed);
    s.ends[i] = gPoints[i].ends.load(std::memory_order_relaxed);
  }
}

// One experiment as a block of lines, written with one append so that several processes can share the file.
int64_t writeExperiment(const Func& f, int percent, const Snapshot& a, const Snapshot& b, int64_t selectedSamples) {
  const int64_t real = b.ns - a.ns, paused = b.owed - a.owed;
  std::string out;
  char line[1400];
  snprintf(line, sizeof(line), "experiment\tselected=%s\tspeedup=%.2f\tduration=%lld\tselected-samples=%lld\treal-duration=%lld\tpaused=%lld\tpid=%d\n", f.name.c_str(),
           percent / 100.0, (long long)(real - paused), (long long)selectedSamples, (long long)real, (long long)paused, (int)getpid());
  out += line;
  int64_t fewest = -1;
  for (int i = 0; i < kMaxPoints; i++) {
    const char* name = gPoints[i].name.load(std::memory_order_acquire);
    if (!name) continue;
    const int64_t dv = b.visits[i] - a.visits[i], db = b.begins[i] - a.begins[i], de = b.ends[i] - a.ends[i];
    if (dv > 0 || (db == 0 && de == 0)) {
      snprintf(line, sizeof(line), "throughput-point\tname=%s\tdelta=%lld\n", name, (long long)dv);
      out += line;
      if (fewest < 0 || dv < fewest) fewest = dv;
    }
    if (db > 0 || de > 0) {
      snprintf(line, sizeof(line), "latency-point\tname=%s\tarrivals=%lld\tdepartures=%lld\tdifference=%lld\n", name, (long long)db, (long long)de,
               (long long)(b.begins[i] - b.ends[i]));
      out += line;
      if (fewest < 0 || de < fewest) fewest = de;
    }
  }
  const int fd = open(gCfg->file.c_str(), O_WRONLY | O_CREAT | O_APPEND | O_CLOEXEC, 0644);
  if (fd >= 0) {
    ssize_t w = write(fd, out.data(), out.size());
    (void)w;
    close(fd);
  }
  gDone.fetch_add(1);
  return fewest;
}

void beginExperiment(const Func& f, int percent, Snapshot& at) {
  gExp.selected.store(f.entry);
  gExp.percent.store(percent);
  gExp.selectedSamples.store(0);
  snapshot(at);
  gExp.running.store(true, std::memory_order_release);
  if (gCfg->verbose)
    fprintf(stderr, "[b200causal] Starting causal experiment #%llu: %s at %d %% -> %s\n", (unsigned long long)gDone.load() + 1, f.name.c_str(), percent, gCfg->file.c_str());
}
void endExperiment(const Func& f, int percent, const Snapshot& from, int64_t* fewest = nullptr) {
  gExp.running.store(false, std::memory_order_release);
  Snapshot to;
  snapshot(to);
  const int64_t few = writeExperiment(f, percent, from, to, gExp.selectedSamples.load());
  if (fewest) *fewest = few;
}

// Sleeps in short steps so that stopping does not have to wait for a whole experiment.
bool napUnlessStopping(double seconds) {
  const int64_t until = monoNs() + (int64_t)(seconds * 1e9);
  while (!gStopping.load(std::memory_order_relaxed)) {
    const int64_t left = until - monoNs();
    if (left <= 0) return true;
    pauseNs(std::min<int64_t>(left, 20000000));
  }
  return false;
}

int drawSpeedup(std::mt19937_64& rng) {
  const auto& s = gCfg->speedups;
  const bool hasZero = std::find(s.begin(), s.end(), 0) != s.end();
  if (hasZero && s.size() > 1 && rng() % 4 == 0) return 0;  // the baseline is what everything is compared with: draw it more often
  return s[rng() % s.size()];
}

Func* gFixed = nullptr;  // end-to-end: the one experiment of the run (a pointer: the load-time start runs before this file's objects are built)
int gFixedPercent = 0;
Snapshot* gFixedFrom = nullptr;

void* controllerMain(void*) {
  gControllerTid = (pid_t)syscall(SYS_gettid);
  std::mt19937_64 rng(gCfg->seed ? gCfg->seed : (uint64_t)monoNs() ^ ((uint64_t)getpid() << 32));
  if (!napUnlessStopping(gCfg->delaySeconds)) return nullptr;
  const int64_t t0 = monoNs();
  double length = gCfg->experimentSeconds;
  uint64_t seen = gRecentNext.load();
  while (!gStopping.load()) {
    if (gCfg->durationSeconds > 0 && (monoNs() - t0) > (int64_t)(gCfg->durationSeconds * 1e9)) break;
    // The target: the function of a sample taken since the previous experiment ended.
    const uint64_t now = gRecentNext.load();
    if (now == seen) {
      if (!napUnlessStopping(0.01)) break;
      continue;
    }
    const uint64_t span = std::min<uint64_t>(now - seen, kRecent);
    const int idx = gRecent[(now - 1 - rng() % span) % kRecent].load();
    if (idx < 0 || idx >= (int)gFuncs->size()) { seen = now; continue; }
    const Func& f = (*gFuncs)[idx];
    const int percent = drawSpeedup(rng);
    Snapshot from;
    beginExperiment(f, percent, from);
    napUnlessStopping(length);
    int64_t fewest = -1;
    endExperiment(f, percent, from, &fewest);
    // Too few visits make a noisy rate (an experiment sees a whole number of them: with N visits the rate is only good to
    // 1 / N): lengthen; plenty: shorten again.
    if (fewest >= 0 && fewest < 10 && length < 8.0) length *= 2;
    else if (fewest >= 40 && length > gCfg->experimentSeconds) length /= 2;
    if (!napUnlessStopping(std::min(length / 2, 0.25))) break;  // the threads serve what is still owed before the next baseline
    seen = gRecentNext.load();
  }
  return nullptr;
}

std::vector<int> parseSpeedups(const char* s) {
  std::vector<int> out;
  for (const char* p = s ? s : ""; *p;) {
    char* end = nullptr;
    const long v = strtol(p, &end, 10);
    if (end == p) { p++; continue; }
    if (v >= 0 && v <= 100) out.push_back((int)v);
    p = end;
  }
  return out;
}

char gEnvFile[1024] = "";
void atExitStop() { b200causalStop(); }
void inChild() {  // neither the timer nor the controller thread survives a fork
  gActive.store(false);
  gExp.running.store(false);
  gControllerUp = false;
}

__attribute__((constructor)) void onLoad() {
  pthread_atfork(nullptr, nullptr, inChild);
  const char* file = getenv("B200CAUSAL_FILE");
  if (!file || !*file) return;
  snprintf(gEnvFile, sizeof(gEnvFile), "%s", file);
  auto num = [](const char* name, double dflt) { const char* v = getenv(name); return v && *v ? atof(v) : dflt; };
  b200causalConfig_t c;
  memset(&c, 0, sizeof(c));
  c.file = gEnvFile;
  c.binaryScope = getenv("B200CAUSAL_BINARY_SCOPE");
  c.functionScope = getenv("B200CAUSAL_FUNCTION_SCOPE");
  c.functionExclude = getenv("B200CAUSAL_FUNCTION_EXCLUDE");
  c.speedups = getenv("B200CAUSAL_FIXED_SPEEDUP");
  c.sourceRanges = getenv("B200CAUSAL_SOURCE_RANGES");
  c.backend = getenv("B200CAUSAL_BACKEND");
  c.freqHz = num("B200CAUSAL_FREQ", 1000.0);
  c.experimentSeconds = num("B200CAUSAL_EXPERIMENT_SECONDS", 0.5);
  c.delaySeconds = num("B200CAUSAL_DELAY", 0.0);
  c.durationSeconds = num("B200CAUSAL_DURATION", 0.0);
  c.endToEnd = num("B200CAUSAL_END_TO_END", 0) != 0;
  c.resetFile = num("B200CAUSAL_FILE_RESET", 0) != 0;
  c.seed = (uint64_t)num("B200CAUSAL_RANDOM_SEED", 0);
  c.verbose = num("B200CAUSAL_VERBOSE", 0) != 0;
  const int rc = b200causalStart(&c);
  if (rc == 0) atexit(atExitStop);
  else fprintf(stderr, "[b200causal] not started (%d)\n", rc);
}

}  // namespace

extern "C" {

int b200causalStart(const b200causalConfig_t* cfg) {
  if (gActive.load()) return -1;
  if (!cfg || !cfg->file || !*cfg->file) return -2;
  const double freq = cfg->freqHz > 0 ? cfg->freqHz : 1000.0;
  if (freq > 10000.0 || cfg->experimentSeconds < 0 || cfg->delaySeconds < 0) return -2;
  // Functions in scope.
  ScopeArgs scope;
  const char* bin = (cfg->binaryScope && *cfg->binaryScope) ? cfg->binaryScope : "%MAIN%";
  scope.mainOnly = !strcmp(bin, "%MAIN%");
  if (!scope.mainOnly) scope.binary = regexList(bin);
  scope.function = regexList(cfg->functionScope);
  scope.exclude = regexList(cfg->functionExclude);
  scope.exclude.emplace_back("^_|::_M");  // runtime and standard-library internals are never what one wants to speed up
  if (cfg->sourceRanges && *cfg->sourceRanges) {
    if (!readSourceRanges(cfg->sourceRanges, scope.found)) return -2;
  } else {
    dl_iterate_phdr(onObject, &scope);
  }
  std::sort(scope.found.begin(), scope.found.end(), [](const Func& a, const Func& b) { return a.lo < b.lo || (a.lo == b.lo && a.hi > b.hi); });
  auto* funcs = new std::vector<Func>();
  for (auto& f : scope.found)
    if (funcs->empty() || f.lo >= funcs->back().hi) funcs->push_back(std::move(f));  // aliases and overlaps: keep the first
  if (funcs->empty()) { delete funcs; return -3; }
  for (size_t i = 0; i < funcs->size(); i++)
    if ((*funcs)[i].entry < 0) (*funcs)[i].entry = (int)i;  // a function is its own entry; source lines came with theirs
  delete gFuncs;
  gFuncs = funcs;
  delete gCfg;
  gCfg = new Config();
  gCfg->file = cfg->file;
  gCfg->speedups = parseSpeedups(cfg->speedups);
  if (gCfg->speedups.empty()) gCfg->speedups = {0, 10, 20, 30, 40, 50, 60, 70, 80, 90, 100};
  gCfg->freqHz = freq;
  gCfg->experimentSeconds = cfg->experimentSeconds > 0 ? cfg->experimentSeconds : 0.5;
  gCfg->delaySeconds = cfg->delaySeconds;
  gCfg->durationSeconds = cfg->durationSeconds;
  gCfg->endToEnd = cfg->endToEnd != 0;
  gCfg->verbose = cfg->verbose != 0;
  gCfg->seed = cfg->seed;
  gCfg->backend = (cfg->backend && *cfg->backend) ? cfg->backend : "auto";
  if (gCfg->backend != "auto" && gCfg->backend != "perf" && gCfg->backend != "timer") return -2;
  if (cfg->resetFile) {
    const int fd = open(cfg->file, O_WRONLY | O_CREAT | O_TRUNC | O_CLOEXEC, 0644);
    if (fd >= 0) close(fd);
  }
  if (!gKeyMade) gKeyMade = pthread_key_create(&gKey, onThreadExit) == 0;
  void* warm[4];
  backtrace(warm, 4);  // loads the unwinder now, not inside the first signal
  for (auto& r : gRecent) r.store(-1);
  gRecentNext.store(0);
  gStopping.store(false);
  gStartNs = monoNs();
  {
    char line[96];
    const int n = snprintf(line, sizeof(line), "startup\ttime=%lld\n", (long long)gStartNs);
    const int fd = open(cfg->file, O_WRONLY | O_CREAT | O_APPEND | O_CLOEXEC, 0644);
    if (fd < 0) return -2;
    ssize_t w = write(fd, line, n);
    (void)w;
    close(fd);
  }
  struct sigaction sa;
  memset(&sa, 0, sizeof(sa));
  sa.sa_sigaction = onSample;
  sa.sa_flags = SA_SIGINFO | SA_RESTART;
  sigemptyset(&sa.sa_mask);
  if (sigaction(SIGPROF, &sa, &gOldAction) != 0) return -4;
  gActive.store(true);
  if (gCfg->endToEnd) {
    std::mt19937_64 rng(gCfg->seed ? gCfg->seed : (uint64_t)monoNs() ^ ((uint64_t)getpid() << 32));
    delete gFixed;
    gFixed = new Func((*gFuncs)[rng() % gFuncs->size()]);
    gFixedPercent = gCfg->speedups[rng() % gCfg->speedups.size()];
    delete gFixedFrom;
    gFixedFrom = new Snapshot();
    beginExperiment(*gFixed, gFixedPercent, *gFixedFrom);
  } else {
    if (pthread_create(&gController, nullptr, controllerMain, nullptr) != 0) { gActive.store(false); return -4; }
    gControllerUp = true;
  }
  gPerf.store(false);
  if (gCfg->backend != "timer") {
    gPerfPeriodNs = std::max<int64_t>(50000, (int64_t)(1e9 / freq));
    gPerf.store(true);  // before the first event is armed: its handler has to arm it again
    if (openPerfForExistingThreads()) {
      if (gCfg->verbose) fprintf(stderr, "[b200causal] samples from per-thread CPU-clock events every %lld us\n", (long long)(gPerfPeriodNs / 1000));
      return 0;
    }
    gPerf.store(false);
    if (gCfg->backend == "perf") {
      fprintf(stderr, "[b200causal] per-thread CPU-clock events are not available here (perf_event_open: %s)\n", strerror(errno));
      b200causalStop();
      return -4;
    }
  }
  if (gCfg->verbose) fprintf(stderr, "[b200causal] samples from the process CPU-time timer (scheduler-tick granularity)\n");
  const long us = std::max(1L, (long)(1e6 / freq));
  itimerval tv;
  tv.it_interval.tv_sec = us / 1000000;
  tv.it_interval.tv_usec = us % 1000000;
  tv.it_value = tv.it_interval;
  if (setitimer(ITIMER_PROF, &tv, nullptr) != 0) {
    b200causalStop();
    return -4;
  }
  return 0;
}

int b200causalStop(void) {
  if (!gActive.load()) return 0;
  gStopping.store(true);
  itimerval tv;
  memset(&tv, 0, sizeof(tv));
  setitimer(ITIMER_PROF, &tv, nullptr);
  closePerf();
  if (gControllerUp) {
    void* r = nullptr;
    pthread_join(gController, &r);  // ends and writes the experiment it was in
    gControllerUp = false;
  }
  if (gCfg && gCfg->endToEnd && gFixed && gFixedFrom && gExp.running.load()) endExperiment(*gFixed, gFixedPercent, *gFixedFrom);
  gActive.store(false);
  // Signals already queued still arrive: the handler stays installed and returns at once while not active.
  for (int i = 0; i < 1000 && gInHandler.load(std::memory_order_acquire) != 0; i++) usleep(1000);
  if (gCfg) {
    char line[128];
    const int n = snprintf(line, sizeof(line), "runtime\ttime=%lld\tsamples=%lld\n", (long long)(monoNs() - gStartNs), (long long)gSamples.load());
    const int fd = open(gCfg->file.c_str(), O_WRONLY | O_CREAT | O_APPEND | O_CLOEXEC, 0644);
    if (fd >= 0) {
      ssize_t w = write(fd, line, n);
      (void)w;
      close(fd);
    }
  }
  return 0;
}

int b200causalActive(void) { return gActive.load() ? 1 : 0; }
uint64_t b200causalExperiments(void) { return gDone.load(); }

void b200causalProgress(const char* name) {
  if (Point* p = pointFor(name)) p->visits.fetch_add(1, std::memory_order_relaxed);
}
void b200causalBegin(const char* name) {
  if (Point* p = pointFor(name)) p->begins.fetch_add(1, std::memory_order_relaxed);
}
void b200causalEnd(const char* name) {
  if (Point* p = pointFor(name)) p->ends.fetch_add(1, std::memory_order_relaxed);
}

// ---------------------------------------------------------------- the pthread calls that block or wake
// Each wrapper finds the next definition of its name once (the versioned one where the C library has two), does the
// bookkeeping only while sampling is on, and otherwise is a plain call through a pointer.
#define REAL(ret, name, version, ...)                                                       \
  static ret (*real)(__VA_ARGS__) = nullptr;                                                \
  if (!real) {                                                                              \
    void* f = version[0] ? dlvsym(RTLD_NEXT, #name, version) : nullptr;                     \
    if (!f) f = dlsym(RTLD_NEXT, #name);                                                    \
    real = (ret(*)(__VA_ARGS__))f;                                                          \
  }

int pthread_mutex_lock(pthread_mutex_t* m) {
  Thread* t = beforeBlock();
  const int rc = __pthread_mutex_lock(m);
  afterBlock(t, rc == 0);
  return rc;
}
int pthread_mutex_unlock(pthread_mutex_t* m) {
  beforeWake();
  return __pthread_mutex_unlock(m);
}
int pthread_cond_wait(pthread_cond_t* c, pthread_mutex_t* m) {
  REAL(int, pthread_cond_wait, "GLIBC_2.3.2", pthread_cond_t*, pthread_mutex_t*)
  beforeWake();  // the wait releases the mutex
  Thread* t = beforeBlock();
  const int rc = real(c, m);
  afterBlock(t, rc == 0);
  return rc;
}
int pthread_cond_timedwait(pthread_cond_t* c, pthread_mutex_t* m, const timespec* ts) {
  REAL(int, pthread_cond_timedwait, "GLIBC_2.3.2", pthread_cond_t*, pthread_mutex_t*, const timespec*)
  beforeWake();
  Thread* t = beforeBlock();
  const int rc = real(c, m, ts);
  afterBlock(t, rc == 0);  // a wait that timed out was not woken by anybody: it still owes
  return rc;
}
int pthread_cond_clockwait(pthread_cond_t* c, pthread_mutex_t* m, clockid_t clk, const timespec* ts) {
  REAL(int, pthread_cond_clockwait, "", pthread_cond_t*, pthread_mutex_t*, clockid_t, const timespec*)
  beforeWake();
  Thread* t = beforeBlock();
  const int rc = real(c, m, clk, ts);
  afterBlock(t, rc == 0);
  return rc;
}
int pthread_cond_signal(pthread_cond_t* c) {
  REAL(int, pthread_cond_signal, "GLIBC_2.3.2", pthread_cond_t*)
  beforeWake();
  return real(c);
}
int pthread_cond_broadcast(pthread_cond_t* c) {
  REAL(int, pthread_cond_broadcast, "GLIBC_2.3.2", pthread_cond_t*)
  beforeWake();
  return real(c);
}
int pthread_join(pthread_t th, void** ret) {
  REAL(int, pthread_join, "", pthread_t, void**)
  Thread* t = beforeBlock();
  const int rc = real(th, ret);
  afterBlock(t, rc == 0);
  return rc;
}
int pthread_barrier_wait(pthread_barrier_t* b) {
  REAL(int, pthread_barrier_wait, "", pthread_barrier_t*)
  beforeWake();
  Thread* t = beforeBlock();
  const int rc = real(b);
  afterBlock(t, rc == 0 || rc == PTHREAD_BARRIER_SERIAL_THREAD);
  return rc;
}
int sem_wait(sem_t* s) {
  REAL(int, sem_wait, "", sem_t*)
  Thread* t = beforeBlock();
  const int rc = real(s);
  afterBlock(t, rc == 0);
  return rc;
}
int sem_timedwait(sem_t* s, const timespec* ts) {
  REAL(int, sem_timedwait, "", sem_t*, const timespec*)
  Thread* t = beforeBlock();
  const int rc = real(s, ts);
  afterBlock(t, rc == 0);
  return rc;
}
int sem_clockwait(sem_t* s, clockid_t clk, const timespec* ts) {
  REAL(int, sem_clockwait, "", sem_t*, clockid_t, const timespec*)
  Thread* t = beforeBlock();
  const int rc = real(s, clk, ts);
  afterBlock(t, rc == 0);
  return rc;
}
int sem_post(sem_t* s) {
  REAL(int, sem_post, "", sem_t*)
  beforeWake();
  return real(s);
}

// A new thread starts level with its parent (which serves what it owes first: creating a thread wakes it).
struct StartArgs {
  void* (*fn)(void*);
  void* arg;
  int64_t inherit;
};
static void* startThread(void* p) {
  StartArgs a = *(StartArgs*)p;
  free(p);
  if (gActive.load()) {
    Thread* t = keyed(mySlot(a.inherit));
    if (t && gPerf.load() && t->perfFd < 0) t->perfFd = openCpuClock((pid_t)syscall(SYS_gettid));
  }
  return a.fn(a.arg);
}
int pthread_create(pthread_t* th, const pthread_attr_t* attr, void* (*fn)(void*), void* arg) {
  REAL(int, pthread_create, "", pthread_t*, const pthread_attr_t*, void* (*)(void*), void*)
  if (!gActive.load(std::memory_order_relaxed)) return real(th, attr, fn, arg);
  Thread* t = keyed(mySlot());
  serve(t);
  auto* a = (StartArgs*)malloc(sizeof(StartArgs));
  if (!a) return real(th, attr, fn, arg);
  a->fn = fn;
  a->arg = arg;
  a->inherit = t ? t->local.load() : -1;
  const int rc = real(th, attr, startThread, a);
  if (rc != 0) free(a);
  return rc;
}

}  // extern "C"
