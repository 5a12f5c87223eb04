// Plays the part of the Kokkos runtime for the tools-library test: loads the library named on the command line the way
// Kokkos loads KOKKOS_TOOLS_LIBS (dlopen, one dlsym per callback) and drives a small program's worth of callbacks.
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <thread>

struct SpaceHandle { char name[64]; };
struct ToolSettings { bool requires_global_fencing; bool padding[255]; };

template <class F>
F sym(void* h, const char* name) {
  F f = (F)dlsym(h, name);
  if (!f) { fprintf(stderr, "missing %s\n", name); }
  return f;
}

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  void* h = dlopen(argv[1], RTLD_NOW | RTLD_LOCAL);
  if (!h) { fprintf(stderr, "%s\n", dlerror()); return 3; }
  auto settings = sym<void (*)(uint32_t, ToolSettings*)>(h, "kokkosp_request_tool_settings");
  auto init = sym<void (*)(int, uint64_t, uint32_t, void*)>(h, "kokkosp_init_library");
  auto fini = sym<void (*)()>(h, "kokkosp_finalize_library");
  auto bfor = sym<void (*)(const char*, uint32_t, uint64_t*)>(h, "kokkosp_begin_parallel_for");
  auto efor = sym<void (*)(uint64_t)>(h, "kokkosp_end_parallel_for");
  auto bred = sym<void (*)(const char*, uint32_t, uint64_t*)>(h, "kokkosp_begin_parallel_reduce");
  auto ered = sym<void (*)(uint64_t)>(h, "kokkosp_end_parallel_reduce");
  auto bscan = sym<void (*)(const char*, uint32_t, uint64_t*)>(h, "kokkosp_begin_parallel_scan");
  auto escan = sym<void (*)(uint64_t)>(h, "kokkosp_end_parallel_scan");
  auto bfence = sym<void (*)(const char*, uint32_t, uint64_t*)>(h, "kokkosp_begin_fence");
  auto efence = sym<void (*)(uint64_t)>(h, "kokkosp_end_fence");
  auto push = sym<void (*)(const char*)>(h, "kokkosp_push_profile_region");
  auto pop = sym<void (*)()>(h, "kokkosp_pop_profile_region");
  auto mksec = sym<void (*)(const char*, uint32_t*)>(h, "kokkosp_create_profile_section");
  auto startsec = sym<void (*)(uint32_t)>(h, "kokkosp_start_profile_section");
  auto stopsec = sym<void (*)(uint32_t)>(h, "kokkosp_stop_profile_section");
  auto rmsec = sym<void (*)(uint32_t)>(h, "kokkosp_destroy_profile_section");
  auto event = sym<void (*)(const char*)>(h, "kokkosp_profile_event");
  auto bcopy = sym<void (*)(SpaceHandle, const char*, const void*, SpaceHandle, const char*, const void*, uint64_t)>(h, "kokkosp_begin_deep_copy");
  auto ecopy = sym<void (*)()>(h, "kokkosp_end_deep_copy");
  auto alloc = sym<void (*)(SpaceHandle, const char*, const void*, uint64_t)>(h, "kokkosp_allocate_data");
  auto dealloc = sym<void (*)(SpaceHandle, const char*, const void*, uint64_t)>(h, "kokkosp_deallocate_data");
  if (!settings || !init || !fini || !bfor || !efor || !bred || !ered || !bscan || !escan || !bfence || !efence || !push || !pop || !mksec || !startsec ||
      !stopsec || !rmsec || !event || !bcopy || !ecopy || !alloc || !dealloc)
    return 4;
  ToolSettings ts;
  memset(&ts, 1, sizeof(ts));
  settings(1, &ts);
  if (ts.requires_global_fencing) return 5;
  init(0, 20211015, 0, nullptr);
  SpaceHandle host{}, dev{};
  strcpy(host.name, "Host");
  strcpy(dev.name, "Cuda");
  int x = 0;
  alloc(dev, "field", &x, 4096);
  push("timestep");
  uint64_t k1 = 0, k2 = 0, k3 = 0, f1 = 0;
  bfor("axpy", 0, &k1);
  bred("dot", 0, &k2);        // overlaps the parallel_for and ends first
  ered(k2);
  std::thread other([&] { efor(k1); });  // a region may end on another thread
  other.join();
  bscan("prefix", 0, &k3);
  escan(k3);
  bfence("Kokkos::fence after axpy", 0, &f1);
  efence(f1);
  bcopy(host, "field_mirror", &x, dev, "field", &x, 4096);
  ecopy();
  uint32_t sec = 0;
  mksec("solver", &sec);
  startsec(sec);
  event("converged");
  stopsec(sec);
  rmsec(sec);
  pop();
  dealloc(dev, "field", &x, 4096);
  uint32_t open = 0;
  mksec("left open", &open);
  startsec(open);             // closed by finalize
  fini();
  printf("ids %llu %llu %llu %llu\n", (unsigned long long)k1, (unsigned long long)k2, (unsigned long long)k3, (unsigned long long)f1);
  return 0;
}
