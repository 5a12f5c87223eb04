// libb200kokkosp.so — a Kokkos Tools library: name it in KOKKOS_TOOLS_LIBS and every parallel_for / parallel_reduce /
// parallel_scan, fence, deep copy, profile region, profile section and profile event of a Kokkos program becomes a b200tx
// range or marker, next to the kernel, copy and collective records of the other tracers (run the program under
// `tools/prof.py --marker-trace ...`, or set B200COLL_TRACE=1 and B200COLL_TRACE_FILE=<prefix>).
//
// Counterpart of the reference's Kokkos connectors (rocprofiler-sdk source/lib/rocprofiler-sdk-tool/kokkosp/kokkosp.cpp,
// which turns the same callbacks into roctx ranges; rocprofiler-systems source/lib/rocprof-sys/library/kokkosp.cpp). Two
// differences in how the callbacks map: kernels and fences use start/stop ranges keyed by the id that Kokkos hands back
// to the matching end callback, so a region that ends on another thread still closes the right range; and the kind of
// construct is part of the name ("parallel_for: axpy"), so the statistics group them.
//
// The marker entry points are looked up at run time: in the process if the collective library is already loaded, else in
// libb200coll.so beside this file. Without them every callback returns at once.
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <string>

namespace {

struct Api {
  void (*mark)(const char*) = nullptr;
  int (*push)(const char*) = nullptr;
  int (*pop)() = nullptr;
  uint64_t (*start)(const char*) = nullptr;
  void (*stop)(uint64_t) = nullptr;
  void (*enable)(int) = nullptr;
  bool ok = false;
};
Api gApi;
bool gMemoryEvents = false;

void* lookup(void* handle, const char* name) { return handle ? dlsym(handle, name) : nullptr; }

void resolve() {
  void* h = RTLD_DEFAULT;
  if (!dlsym(RTLD_DEFAULT, "b200txRangePush")) {
    h = nullptr;
    Dl_info me;
    if (dladdr((void*)&resolve, &me) && me.dli_fname) {
      std::string dir = me.dli_fname;
      const size_t slash = dir.rfind('/');
      dir = slash == std::string::npos ? "." : dir.substr(0, slash);
      h = dlopen((dir + "/libb200coll.so").c_str(), RTLD_NOW | RTLD_GLOBAL);
    }
    if (!h) h = dlopen("libb200coll.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
      fprintf(stderr, "[b200kokkosp] libb200coll.so not found (%s): Kokkos regions are not recorded\n", dlerror());
      return;
    }
  }
  gApi.mark = (void (*)(const char*))lookup(h, "b200txMark");
  gApi.push = (int (*)(const char*))lookup(h, "b200txRangePush");
  gApi.pop = (int (*)())lookup(h, "b200txRangePop");
  gApi.start = (uint64_t(*)(const char*))lookup(h, "b200txRangeStart");
  gApi.stop = (void (*)(uint64_t))lookup(h, "b200txRangeStop");
  gApi.enable = (void (*)(int))lookup(h, "b200txEnable");
  gApi.ok = gApi.mark && gApi.push && gApi.pop && gApi.start && gApi.stop;
}

std::string label(const char* kind, const char* name) { return std::string(kind) + ": " + (name ? name : ""); }

struct Section {
  std::string name;
  uint64_t open = 0;
};
std::mutex gMu;
std::map<uint32_t, Section> gSections;
uint32_t gNextSection = 1;

// What Kokkos passes for a memory space.
struct SpaceHandle {
  char name[64];
};
struct ToolSettings {
  bool requires_global_fencing;
  bool padding[255];
};

}  // namespace

extern "C" {

void kokkosp_request_tool_settings(const uint32_t, ToolSettings* settings) {
  if (settings) settings->requires_global_fencing = false;  // ranges bracket the host side; device times come from the activity tracer
}

void kokkosp_init_library(const int loadSeq, const uint64_t interfaceVer, const uint32_t, void*) {
  resolve();
  const char* mem = getenv("B200KOKKOSP_MEMORY_EVENTS");
  gMemoryEvents = mem && atoi(mem) != 0;
  const char* verbose = getenv("B200KOKKOSP_VERBOSE");
  if (verbose && atoi(verbose))
    fprintf(stderr, "[b200kokkosp] loaded (sequence %d, interface %llu), markers %s\n", loadSeq, (unsigned long long)interfaceVer, gApi.ok ? "on" : "unavailable");
}

void kokkosp_finalize_library() {
  std::lock_guard<std::mutex> lk(gMu);
  for (auto& kv : gSections)
    if (kv.second.open && gApi.ok) gApi.stop(kv.second.open);
  gSections.clear();
}

#define B200_KERNEL_HOOKS(kind)                                                                   \
  void kokkosp_begin_##kind(const char* name, const uint32_t, uint64_t* kID) {                    \
    const uint64_t id = gApi.ok ? gApi.start(label(#kind, name).c_str()) : 0;                     \
    if (kID) *kID = id;                                                                           \
  }                                                                                               \
  void kokkosp_end_##kind(const uint64_t kID) {                                                   \
    if (gApi.ok && kID) gApi.stop(kID);                                                           \
  }
B200_KERNEL_HOOKS(parallel_for)
B200_KERNEL_HOOKS(parallel_reduce)
B200_KERNEL_HOOKS(parallel_scan)
B200_KERNEL_HOOKS(fence)
#undef B200_KERNEL_HOOKS

void kokkosp_push_profile_region(const char* name) {
  if (gApi.ok) gApi.push(name ? name : "");
}
void kokkosp_pop_profile_region() {
  if (gApi.ok) gApi.pop();
}

void kokkosp_create_profile_section(const char* name, uint32_t* secid) {
  std::lock_guard<std::mutex> lk(gMu);
  const uint32_t id = gNextSection++;
  gSections[id].name = label("section", name);
  if (secid) *secid = id;
}
void kokkosp_start_profile_section(const uint32_t secid) {
  std::lock_guard<std::mutex> lk(gMu);
  auto it = gSections.find(secid);
  if (it == gSections.end() || it->second.open || !gApi.ok) return;
  it->second.open = gApi.start(it->second.name.c_str());
}
void kokkosp_stop_profile_section(const uint32_t secid) {
  std::lock_guard<std::mutex> lk(gMu);
  auto it = gSections.find(secid);
  if (it == gSections.end() || !it->second.open) return;
  if (gApi.ok) gApi.stop(it->second.open);
  it->second.open = 0;
}
void kokkosp_destroy_profile_section(const uint32_t secid) {
  std::lock_guard<std::mutex> lk(gMu);
  auto it = gSections.find(secid);
  if (it == gSections.end()) return;
  if (it->second.open && gApi.ok) gApi.stop(it->second.open);
  gSections.erase(it);
}

void kokkosp_profile_event(const char* name) {
  if (gApi.ok) gApi.mark(label("event", name).c_str());
}

void kokkosp_begin_deep_copy(SpaceHandle dstSpace, const char* dstName, const void*, SpaceHandle srcSpace, const char* srcName, const void*, uint64_t size) {
  if (!gApi.ok) return;
  char buf[200];
  snprintf(buf, sizeof(buf), "deep_copy: %.24s %.24s <- %.24s %.24s (%llu B)", dstSpace.name, dstName ? dstName : "", srcSpace.name, srcName ? srcName : "",
           (unsigned long long)size);
  gApi.push(buf);
}
void kokkosp_end_deep_copy() {
  if (gApi.ok) gApi.pop();
}

void kokkosp_allocate_data(SpaceHandle space, const char* name, const void*, uint64_t size) {
  if (!gApi.ok || !gMemoryEvents) return;
  char buf[160];
  snprintf(buf, sizeof(buf), "allocate: %.24s %.48s (%llu B)", space.name, name ? name : "", (unsigned long long)size);
  gApi.mark(buf);
}
void kokkosp_deallocate_data(SpaceHandle space, const char* name, const void*, uint64_t size) {
  if (!gApi.ok || !gMemoryEvents) return;
  char buf[160];
  snprintf(buf, sizeof(buf), "deallocate: %.24s %.48s (%llu B)", space.name, name ? name : "", (unsigned long long)size);
  gApi.mark(buf);
}

}  // extern "C"
