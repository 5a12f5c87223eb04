// b200sample — call-stack sampling of the host threads of any program, with the clock of the other tracers
// (CLOCK_MONOTONIC), so that "where was the CPU while the GPU waited" can be read next to kernel and collective records.
// It plays the part of the reference's sampling mode (rocprofiler-systems source/lib/rocprof-sys/library/sampling.cpp:
// per-thread timers on CPU time and on real time, a backtrace per signal, post-processed into call stacks when the
// program ends; settings ROCPROFSYS_SAMPLING_FREQ / _CPUTIME / _REALTIME, source/lib/core/config.cpp:425-615).
//
// Two clocks:
//   cpu   ITIMER_PROF: the kernel delivers SIGPROF to a thread that is burning CPU, in proportion to the CPU time used;
//         threads that sleep are not sampled.
//   wall  a sampler thread walks /proc/self/task every period and sends SIGPROF to every thread, so that blocked threads
//         (in a lock, a poll, cudaStreamSynchronize) show up with the stack they wait in.
// The handler only calls backtrace() (warmed up at start, so that it does not load anything inside a signal) into a slot
// of a preallocated ring; symbols are resolved when the samples are written.
//
// Two ways in: LD_PRELOAD=libb200sample.so with B200SAMPLE_PREFIX (files <prefix>.<pid>.samples.csv and
// <prefix>.<pid>.folded), B200SAMPLE_FREQ (Hz, default 100), B200SAMPLE_CLOCK (cpu | wall), B200SAMPLE_DELAY (seconds
// before the first sample), B200SAMPLE_DURATION (seconds of sampling, 0 = to the end); or b200sampleStart / Stop / Write
// from the program.
#include <cxxabi.h>
#include <dirent.h>
#include <dlfcn.h>
#include <execinfo.h>
#include <pthread.h>
#include <signal.h>
#include <sys/syscall.h>
#include <sys/time.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "b200coll/sample.h"

namespace {

constexpr int kMaxDepth = 48;
struct Slot {
  uint64_t ns;
  int32_t tid;
  int32_t depth;  // 0: the slot was reserved but not yet filled
  void* pc[kMaxDepth];
};

Slot* gRing = nullptr;
uint64_t gCap = 0;
std::atomic<uint64_t> gNext{0};
std::atomic<uint64_t> gDropped{0};
std::atomic<bool> gRunning{false};
std::atomic<int> gInHandler{0};
int gMode = B200SAMPLE_CPU;
double gFreq = 100.0;
pthread_t gTicker;
bool gTickerUp = false;
struct sigaction gOldAction;
pid_t gSamplerTid = 0;

uint64_t monoNs() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

void onSignal(int, siginfo_t*, void*) {
  if (!gRunning.load(std::memory_order_relaxed)) return;
  const int saved = errno;
  gInHandler.fetch_add(1, std::memory_order_acquire);
  const pid_t tid = (pid_t)syscall(SYS_gettid);
  if (tid != gSamplerTid) {
    const uint64_t i = gNext.fetch_add(1, std::memory_order_relaxed);
    if (i < gCap) {
      Slot& s = gRing[i];
      s.ns = monoNs();
      s.tid = tid;
      const int d = backtrace(s.pc, kMaxDepth);
      __atomic_store_n(&s.depth, d, __ATOMIC_RELEASE);
    } else {
      gDropped.fetch_add(1, std::memory_order_relaxed);
    }
  }
  gInHandler.fetch_sub(1, std::memory_order_release);
  errno = saved;
}

void* tickerMain(void*) {
  gSamplerTid = (pid_t)syscall(SYS_gettid);
  const pid_t pid = getpid();
  const long periodNs = (long)(1e9 / gFreq);
  timespec next;
  clock_gettime(CLOCK_MONOTONIC, &next);
  while (gRunning.load(std::memory_order_relaxed)) {
    next.tv_nsec += periodNs;
    while (next.tv_nsec >= 1000000000L) { next.tv_nsec -= 1000000000L; next.tv_sec++; }
    clock_nanosleep(CLOCK_MONOTONIC, TIMER_ABSTIME, &next, nullptr);
    if (!gRunning.load(std::memory_order_relaxed)) break;
    DIR* d = opendir("/proc/self/task");
    if (!d) continue;
    while (dirent* e = readdir(d)) {
      if (e->d_name[0] < '0' || e->d_name[0] > '9') continue;
      const pid_t tid = (pid_t)atoi(e->d_name);
      if (tid != gSamplerTid) syscall(SYS_tgkill, pid, tid, SIGPROF);
    }
    closedir(d);
  }
  return nullptr;
}

// "outer;...;leaf" of one sample. The two innermost frames are the handler and the signal trampoline.
std::string symbol(void* pc, std::map<void*, std::string>& cache) {
  auto it = cache.find(pc);
  if (it != cache.end()) return it->second;
  std::string out;
  Dl_info info;
  if (dladdr(pc, &info) && info.dli_sname) {
    int status = 0;
    char* dem = abi::__cxa_demangle(info.dli_sname, nullptr, nullptr, &status);
    out = (status == 0 && dem) ? dem : info.dli_sname;
    free(dem);
  } else if (dladdr(pc, &info) && info.dli_fname) {
    const char* base = strrchr(info.dli_fname, '/');
    char buf[512];
    snprintf(buf, sizeof(buf), "%s+0x%lx", base ? base + 1 : info.dli_fname, (unsigned long)((char*)pc - (char*)info.dli_fbase));
    out = buf;
  } else {
    char buf[32];
    snprintf(buf, sizeof(buf), "%p", pc);
    out = buf;
  }
  for (char& c : out)
    if (c == ';' || c == ',' || c == '\n' || c == '"') c = ' ';
  cache[pc] = out;
  return out;
}

std::string folded(const Slot& s, std::map<void*, std::string>& cache) {
  std::string out;
  const int skip = s.depth > 2 ? 2 : 0;
  for (int i = s.depth - 1; i >= skip; i--) {
    if (!out.empty()) out += ';';
    out += symbol(s.pc[i], cache);
  }
  return out;
}

char gPrefix[900] = "";  // plain storage: the load-time constructor below may run before C++ objects of this file are built

void atExitWrite() {
  b200sampleStop();
  if (gPrefix[0]) {
    char path[1024];
    snprintf(path, sizeof(path), "%s.%d", gPrefix, (int)getpid());
    b200sampleWrite(path);
  }
}

// With B200SAMPLE_SIGNALS=1 (the tracing launcher sets it) a program ended by SIGTERM / SIGINT / SIGQUIT / SIGABRT still
// writes its samples, then the signal takes its default course; a handler of the program's own is never replaced.
void onFatalSignal(int sig) {
  static std::atomic<int> once{0};
  if (once.exchange(1) == 0) atExitWrite();
  signal(sig, SIG_DFL);
  raise(sig);
}

void installSignalFlush() {
  const char* v = getenv("B200SAMPLE_SIGNALS");
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

// A forked child starts with an empty ring and no timer (interval timers are not inherited, nor is the sampler thread).
void inChild() {
  gRunning.store(false);
  gTickerUp = false;
  gNext.store(0);
  gDropped.store(0);
}

__attribute__((constructor)) void onLoad() {
  pthread_atfork(nullptr, nullptr, inChild);
  const char* prefix = getenv("B200SAMPLE_PREFIX");
  if (!prefix || !*prefix) return;
  snprintf(gPrefix, sizeof(gPrefix), "%s", prefix);
  const char* f = getenv("B200SAMPLE_FREQ");
  const char* c = getenv("B200SAMPLE_CLOCK");
  const char* d = getenv("B200SAMPLE_DELAY");
  const double freq = f ? atof(f) : 100.0;
  const int mode = (c && !strcmp(c, "wall")) ? B200SAMPLE_WALL : B200SAMPLE_CPU;
  const double delay = d ? atof(d) : 0.0;
  if (b200sampleStartDelayed(freq, mode, delay) == 0) {
    atexit(atExitWrite);
    installSignalFlush();
    // B200SAMPLE_DURATION: sample for this many seconds (after the delay), then stop; the program runs on unsampled and the
    // files are written when it ends (the reference's sampling duration setting, ROCPROFSYS_SAMPLING_DURATION).
    const char* dur = getenv("B200SAMPLE_DURATION");
    static double window = 0.0;
    window = dur ? atof(dur) : 0.0;
    if (window > 0.0) {
      pthread_t th;
      auto body = +[](void* p) -> void* {
        const double seconds = *(double*)p;
        timespec ts{(time_t)seconds, (long)((seconds - (time_t)seconds) * 1e9)};
        while (nanosleep(&ts, &ts) != 0 && errno == EINTR) {
        }
        b200sampleStop();
        return nullptr;
      };
      static double total = 0.0;
      total = window + (mode == B200SAMPLE_CPU ? delay : 0.0);  // wall mode has slept through the delay already
      if (pthread_create(&th, nullptr, body, &total) == 0) pthread_detach(th);
    }
  }
}

}  // namespace

extern "C" {

int b200sampleStartDelayed(double freqHz, int mode, double delaySeconds) {
  if (gRunning.load()) return -1;
  if (!(freqHz > 0.0) || freqHz > 10000.0 || (mode != B200SAMPLE_CPU && mode != B200SAMPLE_WALL) || delaySeconds < 0.0) return -2;
  if (!gRing) {
    const char* cap = getenv("B200SAMPLE_MAX_SAMPLES");
    gCap = cap ? strtoull(cap, nullptr, 10) : (1ull << 18);
    if (gCap < 16) gCap = 16;
    gRing = (Slot*)calloc(gCap, sizeof(Slot));
    if (!gRing) return -3;
  }
  void* warm[4];
  backtrace(warm, 4);  // loads the unwinder now, not inside the first signal
  gMode = mode;
  gFreq = freqHz;
  struct sigaction sa;
  memset(&sa, 0, sizeof(sa));
  sa.sa_sigaction = onSignal;
  sa.sa_flags = SA_SIGINFO | SA_RESTART;
  sigemptyset(&sa.sa_mask);
  if (sigaction(SIGPROF, &sa, &gOldAction) != 0) return -4;
  gRunning.store(true);
  if (mode == B200SAMPLE_CPU) {
    const long us = (long)(1e6 / freqHz);
    itimerval tv;
    tv.it_interval.tv_sec = us / 1000000;
    tv.it_interval.tv_usec = us % 1000000;
    const long first = delaySeconds > 0.0 ? (long)(delaySeconds * 1e6) : us;
    tv.it_value.tv_sec = first / 1000000;
    tv.it_value.tv_usec = first % 1000000;
    if (setitimer(ITIMER_PROF, &tv, nullptr) != 0) { gRunning.store(false); return -5; }
  } else {
    if (delaySeconds > 0.0) usleep((useconds_t)(delaySeconds * 1e6));
    if (pthread_create(&gTicker, nullptr, tickerMain, nullptr) != 0) { gRunning.store(false); return -5; }
    gTickerUp = true;
  }
  return 0;
}

int b200sampleStart(double freqHz, int mode) { return b200sampleStartDelayed(freqHz, mode, 0.0); }

int b200sampleStop(void) {
  if (!gRunning.exchange(false)) return 0;
  if (gMode == B200SAMPLE_CPU) {
    itimerval tv;
    memset(&tv, 0, sizeof(tv));
    setitimer(ITIMER_PROF, &tv, nullptr);
  } else if (gTickerUp) {
    pthread_join(gTicker, nullptr);
    gTickerUp = false;
  }
  // Signals already queued still arrive: the handler stays installed and returns at once while not running.
  for (int i = 0; i < 1000 && gInHandler.load(std::memory_order_acquire) != 0; i++) usleep(1000);
  return 0;
}

uint64_t b200sampleCount(void) {
  const uint64_t n = gNext.load();
  return n < gCap ? n : gCap;
}

uint64_t b200sampleDropped(void) { return gDropped.load(); }

void b200sampleClear(void) {
  if (gRunning.load()) return;
  if (gRing) memset(gRing, 0, gCap * sizeof(Slot));
  gNext.store(0);
  gDropped.store(0);
}

int b200sampleWrite(const char* prefix) {
  if (!prefix || gRunning.load()) return -1;
  const uint64_t n = b200sampleCount();
  std::map<void*, std::string> cache;
  std::map<std::string, uint64_t> counts;
  std::string p1 = std::string(prefix) + ".samples.csv", p2 = std::string(prefix) + ".folded";
  FILE* f = fopen(p1.c_str(), "w");
  if (!f) return -2;
  fprintf(f, "timestamp_ns,tid,depth,clock,stack\n");
  for (uint64_t i = 0; i < n; i++) {
    const Slot& s = gRing[i];
    const int depth = __atomic_load_n(&s.depth, __ATOMIC_ACQUIRE);
    if (depth <= 0) continue;
    const std::string st = folded(s, cache);
    if (st.empty()) continue;
    fprintf(f, "%llu,%d,%d,%s,\"%s\"\n", (unsigned long long)s.ns, s.tid, depth > 2 ? depth - 2 : depth, gMode == B200SAMPLE_CPU ? "cpu" : "wall", st.c_str());
    counts[st]++;
  }
  fclose(f);
  f = fopen(p2.c_str(), "w");
  if (!f) return -2;
  for (auto& kv : counts) fprintf(f, "%s %llu\n", kv.first.c_str(), (unsigned long long)kv.second);
  fclose(f);
  return 2;
}

}  // extern "C"
