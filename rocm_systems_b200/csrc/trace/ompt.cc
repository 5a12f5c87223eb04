// libb200ompt.so — an OpenMP tool (OMPT): name it in OMP_TOOL_LIBRARIES and the parallel regions, implicit tasks,
// worksharing constructs, barriers and target regions (with their data transfers and kernel submissions) of an OpenMP
// program become b200tx ranges and markers, next to the kernel, copy and collective records of the other tracers (run the
// program under `tools/prof.py --openmp-trace ...`, or set B200COLL_TRACE=1 and B200COLL_TRACE_FILE=<prefix>).
//
// Counterpart of the reference's OpenMP support (rocprofiler-sdk source/lib/rocprofiler-sdk/ompt.cpp and ompt/: the OMPT
// callbacks as a tracing domain; rocprofiler-systems source/lib/rocprof-sys/library/ompt.cpp: the same callbacks as
// regions of its timeline). How the callbacks map:
//   parallel begin / end            one start/stop range per region, keyed through the region's tool data word, so the end
//                                   finds its begin whichever thread reports it
//   implicit task, work, masked,    push / pop on the thread that runs them (they nest properly per thread)
//   sync region (barriers, waits)
//   target begin / end              start/stop range keyed by the target id; data operations and kernel submissions of the
//                                   region are markers that carry the id, the direction and the byte count
//   thread begin / end              markers
// The marker entry points are looked up at run time: in the process if the collective library is already loaded, else in
// libb200coll.so beside this file. Without them the tool declines (ompt_start_tool returns NULL) and the runtime carries on
// untraced.
#include <Openmp/omp-tools.h>
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
  bool ok = false;
};
Api gApi;
bool gVerbose = false;

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
    if (!h) return;
  }
  gApi.mark = (void (*)(const char*))dlsym(h, "b200txMark");
  gApi.push = (int (*)(const char*))dlsym(h, "b200txRangePush");
  gApi.pop = (int (*)())dlsym(h, "b200txRangePop");
  gApi.start = (uint64_t(*)(const char*))dlsym(h, "b200txRangeStart");
  gApi.stop = (void (*)(uint64_t))dlsym(h, "b200txRangeStop");
  gApi.ok = gApi.mark && gApi.push && gApi.pop && gApi.start && gApi.stop;
}

const char* workName(ompt_work_t w) {
  switch (w) {
    case ompt_work_loop: return "omp loop";
    case ompt_work_sections: return "omp sections";
    case ompt_work_single_executor: return "omp single";
    case ompt_work_single_other: return "omp single (other)";
    case ompt_work_workshare: return "omp workshare";
    case ompt_work_distribute: return "omp distribute";
    case ompt_work_taskloop: return "omp taskloop";
    default: return "omp work";
  }
}
const char* syncName(ompt_sync_region_t k) {
  switch (k) {
    case ompt_sync_region_barrier: return "omp barrier";
    case ompt_sync_region_barrier_implicit: return "omp implicit barrier";
    case ompt_sync_region_barrier_explicit: return "omp barrier (explicit)";
    case ompt_sync_region_barrier_implementation: return "omp barrier (runtime)";
    case ompt_sync_region_taskwait: return "omp taskwait";
    case ompt_sync_region_taskgroup: return "omp taskgroup";
    case ompt_sync_region_reduction: return "omp reduction";
    default: return "omp sync";
  }
}
const char* targetName(ompt_target_t k) {
  switch (k) {
    case ompt_target: return "omp target";
    case ompt_target_enter_data: return "omp target enter data";
    case ompt_target_exit_data: return "omp target exit data";
    case ompt_target_update: return "omp target update";
    default: return "omp target";
  }
}
const char* dataOpName(ompt_target_data_op_t op) {
  switch (op) {
    case ompt_target_data_alloc: return "alloc";
    case ompt_target_data_transfer_to_device: return "to device";
    case ompt_target_data_transfer_from_device: return "from device";
    case ompt_target_data_delete: return "delete";
    case ompt_target_data_associate: return "associate";
    case ompt_target_data_disassociate: return "disassociate";
    default: return "data op";
  }
}

std::mutex gMu;
std::map<ompt_id_t, uint64_t> gTargets;  // target id -> open range

void onThreadBegin(ompt_thread_t type, ompt_data_t*) {
  gApi.mark(type == ompt_thread_initial ? "omp thread begin (initial)" : type == ompt_thread_worker ? "omp thread begin (worker)" : "omp thread begin");
}
void onThreadEnd(ompt_data_t*) { gApi.mark("omp thread end"); }

void onParallelBegin(ompt_data_t*, const ompt_frame_t*, ompt_data_t* parallel, unsigned requested, int, const void*) {
  char buf[64];
  snprintf(buf, sizeof(buf), "omp parallel (%u threads requested)", requested);
  const uint64_t id = gApi.start(buf);
  if (parallel) parallel->value = id;
}
void onParallelEnd(ompt_data_t* parallel, ompt_data_t*, int, const void*) {
  if (parallel && parallel->value) {
    gApi.stop(parallel->value);
    parallel->value = 0;
  }
}
void onImplicitTask(ompt_scope_endpoint_t ep, ompt_data_t*, ompt_data_t*, unsigned team, unsigned index, int flags) {
  if (flags & ompt_task_initial) return;  // the initial task spans the program: not a region of interest
  if (ep == ompt_scope_begin) {
    char buf[64];
    snprintf(buf, sizeof(buf), "omp implicit task %u/%u", index, team);
    gApi.push(buf);
  } else {
    gApi.pop();
  }
}
void onWork(ompt_work_t w, ompt_scope_endpoint_t ep, ompt_data_t*, ompt_data_t*, uint64_t count, const void*) {
  if (ep == ompt_scope_begin) {
    char buf[80];
    snprintf(buf, sizeof(buf), "%s (%llu)", workName(w), (unsigned long long)count);
    gApi.push(buf);
  } else {
    gApi.pop();
  }
}
void onMaster(ompt_scope_endpoint_t ep, ompt_data_t*, ompt_data_t*, const void*) {
  if (ep == ompt_scope_begin) gApi.push("omp masked");
  else gApi.pop();
}
void onSync(ompt_sync_region_t kind, ompt_scope_endpoint_t ep, ompt_data_t*, ompt_data_t*, const void*) {
  if (ep == ompt_scope_begin) gApi.push(syncName(kind));
  else gApi.pop();
}
void onTarget(ompt_target_t kind, ompt_scope_endpoint_t ep, int device, ompt_data_t*, ompt_id_t id, const void*) {
  std::lock_guard<std::mutex> lk(gMu);
  if (ep == ompt_scope_begin) {
    char buf[80];
    snprintf(buf, sizeof(buf), "%s (device %d, id %llu)", targetName(kind), device, (unsigned long long)id);
    gTargets[id] = gApi.start(buf);
  } else {
    auto it = gTargets.find(id);
    if (it != gTargets.end()) {
      gApi.stop(it->second);
      gTargets.erase(it);
    }
  }
}
void onTargetDataOp(ompt_id_t target, ompt_id_t, ompt_target_data_op_t op, void*, int src, void*, int dst, size_t bytes, const void*) {
  char buf[96];
  snprintf(buf, sizeof(buf), "omp target data %s: %zu B, device %d -> %d (id %llu)", dataOpName(op), bytes, src, dst, (unsigned long long)target);
  gApi.mark(buf);
}
void onTargetSubmit(ompt_id_t target, ompt_id_t, unsigned teams) {
  char buf[80];
  snprintf(buf, sizeof(buf), "omp target submit: %u teams (id %llu)", teams, (unsigned long long)target);
  gApi.mark(buf);
}

int initialize(ompt_function_lookup_t lookup, int, ompt_data_t*) {
  auto set = (ompt_set_callback_t)lookup("ompt_set_callback");
  if (!set) return 0;  // zero: the runtime drops the tool
  int accepted = 0;
  auto reg = [&](ompt_callbacks_t which, ompt_callback_t fn) {
    const ompt_set_result_t r = set(which, fn);
    if (r != ompt_set_error && r != ompt_set_never) accepted++;
  };
  reg(ompt_callback_thread_begin, (ompt_callback_t)onThreadBegin);
  reg(ompt_callback_thread_end, (ompt_callback_t)onThreadEnd);
  reg(ompt_callback_parallel_begin, (ompt_callback_t)onParallelBegin);
  reg(ompt_callback_parallel_end, (ompt_callback_t)onParallelEnd);
  reg(ompt_callback_implicit_task, (ompt_callback_t)onImplicitTask);
  reg(ompt_callback_work, (ompt_callback_t)onWork);
  reg(ompt_callback_master, (ompt_callback_t)onMaster);
  reg(ompt_callback_sync_region, (ompt_callback_t)onSync);
  reg(ompt_callback_target, (ompt_callback_t)onTarget);
  reg(ompt_callback_target_data_op, (ompt_callback_t)onTargetDataOp);
  reg(ompt_callback_target_submit, (ompt_callback_t)onTargetSubmit);
  if (gVerbose) fprintf(stderr, "[b200ompt] %d of 11 callbacks accepted by the OpenMP runtime\n", accepted);
  return 1;
}

void finalize(ompt_data_t*) {
  std::lock_guard<std::mutex> lk(gMu);
  for (auto& kv : gTargets) gApi.stop(kv.second);  // regions the runtime never closed end here
  gTargets.clear();
}

ompt_start_tool_result_t gResult = {initialize, finalize, {0}};

}  // namespace

extern "C" ompt_start_tool_result_t* ompt_start_tool(unsigned int ompVersion, const char* runtimeVersion) {
  const char* v = getenv("B200OMPT_VERBOSE");
  gVerbose = v && atoi(v) != 0;
  resolve();
  if (gVerbose)
    fprintf(stderr, "[b200ompt] OpenMP %u, runtime %s: markers %s\n", ompVersion, runtimeVersion ? runtimeVersion : "?", gApi.ok ? "on" : "unavailable, tool declines");
  return gApi.ok ? &gResult : nullptr;
}
