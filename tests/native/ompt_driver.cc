// Plays the part of an OpenMP runtime for the OMPT tool test: loads the tool the way OMP_TOOL_LIBRARIES is handled (dlopen,
// ompt_start_tool, initialize with a lookup function that offers ompt_set_callback) and then reports the events of a small
// program: a parallel region with two implicit tasks (one on another thread), a loop, a barrier, and a target region with
// a transfer and a kernel submission.
#include <Openmp/omp-tools.h>
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>

#include <thread>

static ompt_callback_t table[64];
static ompt_set_result_t setCallback(ompt_callbacks_t which, ompt_callback_t fn) {
  if ((int)which <= 0 || (int)which >= 64) return ompt_set_error;
  if (which == ompt_callback_master) return ompt_set_never;  // this "runtime" never reports masked regions
  table[which] = fn;
  return ompt_set_always;
}
static ompt_interface_fn_t lookup(const char* name) {
  if (!strcmp(name, "ompt_set_callback")) return (ompt_interface_fn_t)setCallback;
  return nullptr;
}
template <class F>
F cb(ompt_callbacks_t which) { return (F)table[which]; }

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  void* h = dlopen(argv[1], RTLD_NOW | RTLD_LOCAL);
  if (!h) { fprintf(stderr, "%s\n", dlerror()); return 3; }
  auto start = (ompt_start_tool_result_t * (*)(unsigned, const char*)) dlsym(h, "ompt_start_tool");
  if (!start) return 4;
  ompt_start_tool_result_t* tool = start(201811, "stand-in runtime");
  if (!tool) { printf("tool declined\n"); return 0; }
  if (!tool->initialize(lookup, 0, &tool->tool_data)) return 5;
  int set = 0;
  for (auto f : table) set += f != nullptr;
  printf("callbacks %d\n", set);

  ompt_data_t thread0{}, thread1{}, task0{}, par{}, t0{}, t1{};
  cb<ompt_callback_thread_begin_t>(ompt_callback_thread_begin)(ompt_thread_initial, &thread0);
  cb<ompt_callback_implicit_task_t>(ompt_callback_implicit_task)(ompt_scope_begin, nullptr, &task0, 1, 1, ompt_task_initial);  // must be ignored
  cb<ompt_callback_parallel_begin_t>(ompt_callback_parallel_begin)(&task0, nullptr, &par, 2, ompt_parallel_team, nullptr);
  std::thread worker([&] {
    cb<ompt_callback_thread_begin_t>(ompt_callback_thread_begin)(ompt_thread_worker, &thread1);
    cb<ompt_callback_implicit_task_t>(ompt_callback_implicit_task)(ompt_scope_begin, &par, &t1, 2, 1, ompt_task_implicit);
    cb<ompt_callback_work_t>(ompt_callback_work)(ompt_work_loop, ompt_scope_begin, &par, &t1, 500, nullptr);
    cb<ompt_callback_work_t>(ompt_callback_work)(ompt_work_loop, ompt_scope_end, &par, &t1, 500, nullptr);
    cb<ompt_callback_sync_region_t>(ompt_callback_sync_region)(ompt_sync_region_barrier_implicit, ompt_scope_begin, &par, &t1, nullptr);
    cb<ompt_callback_sync_region_t>(ompt_callback_sync_region)(ompt_sync_region_barrier_implicit, ompt_scope_end, &par, &t1, nullptr);
    cb<ompt_callback_implicit_task_t>(ompt_callback_implicit_task)(ompt_scope_end, nullptr, &t1, 2, 1, ompt_task_implicit);
    cb<ompt_callback_thread_end_t>(ompt_callback_thread_end)(&thread1);
  });
  cb<ompt_callback_implicit_task_t>(ompt_callback_implicit_task)(ompt_scope_begin, &par, &t0, 2, 0, ompt_task_implicit);
  cb<ompt_callback_work_t>(ompt_callback_work)(ompt_work_loop, ompt_scope_begin, &par, &t0, 500, nullptr);
  cb<ompt_callback_work_t>(ompt_callback_work)(ompt_work_loop, ompt_scope_end, &par, &t0, 500, nullptr);
  cb<ompt_callback_implicit_task_t>(ompt_callback_implicit_task)(ompt_scope_end, nullptr, &t0, 2, 0, ompt_task_implicit);
  worker.join();
  cb<ompt_callback_parallel_end_t>(ompt_callback_parallel_end)(&par, &task0, ompt_parallel_team, nullptr);
  if (par.value != 0) return 6;  // the tool clears its word when the region ends

  cb<ompt_callback_target_t>(ompt_callback_target)(ompt_target, ompt_scope_begin, 0, &task0, 77, nullptr);
  cb<ompt_callback_target_data_op_t>(ompt_callback_target_data_op)(77, 1, ompt_target_data_transfer_to_device, nullptr, -1, nullptr, 0, 4096, nullptr);
  cb<ompt_callback_target_submit_t>(ompt_callback_target_submit)(77, 2, 148);
  cb<ompt_callback_target_t>(ompt_callback_target)(ompt_target, ompt_scope_end, 0, &task0, 77, nullptr);
  cb<ompt_callback_target_t>(ompt_callback_target)(ompt_target_enter_data, ompt_scope_begin, 1, &task0, 78, nullptr);  // never ended: finalize closes it
  cb<ompt_callback_thread_end_t>(ompt_callback_thread_end)(&thread0);
  tool->finalize(&tool->tool_data);
  printf("ompt driver done\n");
  return 0;
}
