// libb200instr.so — function-level tracing and coverage for code compiled with `-finstrument-functions`: the compiler
// calls __cyg_profile_func_enter / _exit around every function of the translation units built that way, and this library
// turns the calls into (a) per-function statistics: calls, inclusive and exclusive time; (b) marker ranges for calls that
// last at least B200INSTR_MIN_US, so that they show up in the trace next to kernels and collectives; (c) a coverage
// report: which functions of the executable's symbol table were entered at all.
//
// It stands where the reference has binary instrumentation (rocprofiler-systems source/bin/rocprof-sys-instrument inserts
// the same entry / exit calls into an existing binary with Dyninst; source/lib/rocprof-sys/library/coverage.cpp keeps the
// per-function hit counts of its coverage mode). Rewriting binaries is not done here: the instrumentation is the
// compiler's, so it covers what the user rebuilds with the flag (`python -m rocm_systems_b200.tools.instrument flags`).
//
// Ways in: LD_PRELOAD or link the library, set B200INSTR_PREFIX; at exit <prefix>.<pid>.functions.csv and
// <prefix>.<pid>.coverage.json are written. B200INSTR_MIN_US (default 100; negative: no marker ranges),
// B200INSTR_MAX_DEPTH (default 64: deeper calls are counted but not timed separately).
#include <cxxabi.h>
#include <dlfcn.h>
#include <elf.h>
#include <fcntl.h>
#include <link.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <map>
#include <string>
#include <vector>

#define NOINSTR __attribute__((no_instrument_function))

namespace {

constexpr int kSlots = 1 << 15;  // distinct functions that can be told apart
struct Slot {
  std::atomic<void*> fn{nullptr};
  std::atomic<uint64_t> calls{0}, inclusiveNs{0}, exclusiveNs{0};
};
Slot gSlots[kSlots];
std::atomic<uint64_t> gOverflow{0};
std::atomic<bool> gOn{false};
char gPrefix[900] = "";
int64_t gMinNs = 100000;
int gMaxDepth = 64;

struct Frame {
  void* fn;
  uint64_t t0, child;  // entry time; time spent in instrumented callees
};
constexpr int kMaxStack = 256;
__thread Frame tStack[kMaxStack] __attribute__((tls_model("initial-exec")));
__thread int tDepth __attribute__((tls_model("initial-exec"))) = 0;
__thread int tBusy __attribute__((tls_model("initial-exec"))) = 0;  // inside the library: calls it makes are not recorded

uint64_t (*gRangeAt)(const char*, uint64_t, uint64_t) = nullptr;  // the marker library's "a range that is already over"
std::atomic<int> gMarkersLooked{0};

NOINSTR uint64_t nowNs() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

NOINSTR Slot* slotFor(void* fn) {
  uint64_t h = (uint64_t)(uintptr_t)fn;
  h ^= h >> 17;
  h *= 0x9E3779B97F4A7C15ull;
  for (int probe = 0; probe < 64; probe++) {
    Slot& s = gSlots[(h + probe) & (kSlots - 1)];
    void* have = s.fn.load(std::memory_order_acquire);
    if (have == fn) return &s;
    if (!have && s.fn.compare_exchange_strong(have, fn)) return &s;
    if (have == fn) return &s;
  }
  gOverflow.fetch_add(1, std::memory_order_relaxed);
  return nullptr;
}

const std::map<uintptr_t, std::string>& symbols();

NOINSTR std::string nameOf(void* fn) {
  Dl_info info;
  {
    const auto& own = symbols();
    auto it = own.find((uintptr_t)fn);
    if (it != own.end()) return it->second;
  }
  if (dladdr(fn, &info) && info.dli_sname) {
    int status = 0;
    char* d = abi::__cxa_demangle(info.dli_sname, nullptr, nullptr, &status);
    std::string out = (status == 0 && d) ? d : info.dli_sname;
    free(d);
    return out;
  }
  char buf[64];
  if (dladdr(fn, &info) && info.dli_fname) {
    const char* base = strrchr(info.dli_fname, '/');
    snprintf(buf, sizeof(buf), "%.40s+0x%lx", base ? base + 1 : info.dli_fname, (unsigned long)((char*)fn - (char*)info.dli_fbase));
  } else {
    snprintf(buf, sizeof(buf), "%p", fn);
  }
  return buf;
}

NOINSTR void lookMarkers() {
  if (gMarkersLooked.exchange(1)) return;
  gRangeAt = (uint64_t(*)(const char*, uint64_t, uint64_t))dlsym(RTLD_DEFAULT, "b200txRangeAt");
}

// Names (demangled) of the FUNC symbols the executable defines, with their addresses in this process.
NOINSTR int onMain(dl_phdr_info* info, size_t, void* data) {
  auto& out = *(std::map<uintptr_t, std::string>*)data;
  const int fd = open("/proc/self/exe", O_RDONLY | O_CLOEXEC);
  if (fd < 0) return 1;
  struct stat st;
  if (fstat(fd, &st) != 0) { close(fd); return 1; }
  void* map = mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (map == MAP_FAILED) return 1;
  const auto* base = (const unsigned char*)map;
  const auto* eh = (const ElfW(Ehdr)*)base;
  const size_t size = (size_t)st.st_size;
  auto inside = [&](uint64_t off, uint64_t len) { return off <= size && len <= size - off; };
  if (size > sizeof(ElfW(Ehdr)) && memcmp(eh->e_ident, ELFMAG, SELFMAG) == 0 && eh->e_shentsize == sizeof(ElfW(Shdr)) &&
      inside(eh->e_shoff, (uint64_t)eh->e_shnum * sizeof(ElfW(Shdr)))) {
    const auto* sh = (const ElfW(Shdr)*)(base + eh->e_shoff);
    for (int i = 0; i < eh->e_shnum; i++) {
      if (sh[i].sh_type != SHT_SYMTAB || sh[i].sh_link >= eh->e_shnum || !inside(sh[i].sh_offset, sh[i].sh_size)) continue;
      const ElfW(Shdr)& str = sh[sh[i].sh_link];
      if (!inside(str.sh_offset, str.sh_size) || str.sh_size == 0) continue;
      const auto* syms = (const ElfW(Sym)*)(base + sh[i].sh_offset);
      const char* names = (const char*)(base + str.sh_offset);
      for (size_t k = 0; k < sh[i].sh_size / sizeof(ElfW(Sym)); k++) {
        const ElfW(Sym)& s = syms[k];
        if (ELF64_ST_TYPE(s.st_info) != STT_FUNC || s.st_size == 0 || s.st_shndx == SHN_UNDEF || s.st_name >= str.sh_size) continue;
        const char* n = names + s.st_name;
        if (!memchr(n, 0, str.sh_size - s.st_name)) continue;
        int status = 0;
        char* d = abi::__cxa_demangle(n, nullptr, nullptr, &status);
        out[(uintptr_t)info->dlpi_addr + s.st_value] = (status == 0 && d) ? d : n;
        free(d);
      }
    }
  }
  munmap(map, size);
  return 1;  // the executable is the first object
}

// The executable's own functions by address (its symbol table also names the ones that are not exported).
NOINSTR const std::map<uintptr_t, std::string>& symbols() {
  static std::map<uintptr_t, std::string>* m = nullptr;
  if (!m) {
    auto* fresh = new std::map<uintptr_t, std::string>();
    dl_iterate_phdr(onMain, fresh);
    m = fresh;
  }
  return *m;
}

// What coverage is counted over: not the start-up helpers (_start, _init, ...) nor library code instantiated in the program.
NOINSTR bool countsForCoverage(const std::string& name) {
  if (name.empty() || name[0] == '_' || name == "frame_dummy" || name == "register_tm_clones" || name == "deregister_tm_clones") return false;
  const std::string head = name.substr(0, name.find('('));  // without the argument list: a user function may take std:: types
  return head.find("std::") == std::string::npos && head.find("__gnu_cxx::") == std::string::npos;
}

NOINSTR void jsonString(FILE* f, const std::string& s) {
  fputc('"', f);
  for (char c : s) {
    if (c == '"' || c == '\\') fputc('\\', f);
    if ((unsigned char)c >= 0x20) fputc(c, f);
  }
  fputc('"', f);
}

NOINSTR void writeAtExit() {
  if (!gOn.exchange(false) || !gPrefix[0]) return;
  tBusy++;
  struct Row {
    std::string name;
    void* fn;
    uint64_t calls, incl, excl;
  };
  std::vector<Row> rows;
  std::map<uintptr_t, uint64_t> hit;
  for (auto& s : gSlots) {
    void* fn = s.fn.load();
    if (!fn) continue;
    rows.push_back({nameOf(fn), fn, s.calls.load(), s.inclusiveNs.load(), s.exclusiveNs.load()});
    hit[(uintptr_t)fn] = s.calls.load();
  }
  std::sort(rows.begin(), rows.end(), [](const Row& a, const Row& b) { return a.incl > b.incl; });
  char path[1024];
  snprintf(path, sizeof(path), "%s.%d.functions.csv", gPrefix, (int)getpid());
  if (FILE* f = fopen(path, "w")) {
    fprintf(f, "function,calls,inclusive_ns,exclusive_ns\n");
    for (auto& r : rows) {
      std::string n = r.name;
      for (char& c : n)
        if (c == '"') c = '\'';
      fprintf(f, "\"%s\",%llu,%llu,%llu\n", n.c_str(), (unsigned long long)r.calls, (unsigned long long)r.incl, (unsigned long long)r.excl);
    }
    fclose(f);
  }
  size_t called = 0, definedCount = 0;
  std::vector<std::string> uncalled;
  for (auto& kv : symbols()) {
    if (!countsForCoverage(kv.second)) continue;
    definedCount++;
    if (hit.count(kv.first)) called++;
    else uncalled.push_back(kv.second);
  }
  snprintf(path, sizeof(path), "%s.%d.coverage.json", gPrefix, (int)getpid());
  if (FILE* f = fopen(path, "w")) {
    fprintf(f, "{\"functions_defined\": %zu, \"functions_called\": %zu, \"percent\": %.2f, \"distinct_functions_seen\": %zu, \"table_overflow\": %llu,\n \"uncalled\": [",
            definedCount, called, definedCount ? 100.0 * called / definedCount : 0.0, rows.size(), (unsigned long long)gOverflow.load());
    for (size_t i = 0; i < uncalled.size(); i++) {
      if (i) fputs(", ", f);
      jsonString(f, uncalled[i]);
    }
    fprintf(f, "]}\n");
    fclose(f);
  }
  tBusy--;
}

__attribute__((constructor)) NOINSTR void onLoad() {
  const char* p = getenv("B200INSTR_PREFIX");
  if (!p || !*p) return;
  snprintf(gPrefix, sizeof(gPrefix), "%s", p);
  if (const char* v = getenv("B200INSTR_MIN_US")) gMinNs = (int64_t)(atof(v) * 1000.0);
  if (const char* v = getenv("B200INSTR_MAX_DEPTH")) gMaxDepth = std::max(1, std::min(kMaxStack, atoi(v)));
  atexit(writeAtExit);
  gOn.store(true);
}

}  // namespace

extern "C" {

NOINSTR void __cyg_profile_func_enter(void* fn, void*) {
  if (!gOn.load(std::memory_order_relaxed) || tBusy) return;
  const int d = tDepth++;
  if (d >= gMaxDepth || d >= kMaxStack) return;
  tStack[d] = Frame{fn, nowNs(), 0};
}

NOINSTR void __cyg_profile_func_exit(void* fn, void*) {
  if (!gOn.load(std::memory_order_relaxed) || tBusy) return;
  if (tDepth <= 0) return;  // entered before the library was switched on
  const int d = --tDepth;
  if (d >= gMaxDepth || d >= kMaxStack) {
    if (Slot* s = slotFor(fn)) s->calls.fetch_add(1, std::memory_order_relaxed);  // too deep to time: counted for the coverage
    return;
  }
  Frame& fr = tStack[d];
  if (fr.fn != fn) return;  // an exit without its entry (longjmp, an exception through uninstrumented frames): drop it
  const uint64_t t1 = nowNs(), dt = t1 - fr.t0;
  if (Slot* s = slotFor(fn)) {
    s->calls.fetch_add(1, std::memory_order_relaxed);
    s->inclusiveNs.fetch_add(dt, std::memory_order_relaxed);
    s->exclusiveNs.fetch_add(dt > fr.child ? dt - fr.child : 0, std::memory_order_relaxed);
  }
  if (d > 0) tStack[d - 1].child += dt;
  if (gMinNs >= 0 && (int64_t)dt >= gMinNs) {
    // Long enough to be worth a range: recorded after the fact from the two times (the marker library's clock is the same
    // CLOCK_MONOTONIC), and only when that library is in the process.
    tBusy++;
    lookMarkers();
    if (gRangeAt) gRangeAt(nameOf(fn).c_str(), fr.t0, t1);
    tBusy--;
  }
}

}  // extern "C"
