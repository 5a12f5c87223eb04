// Thin per-communicator tracer: one record per collective call with the host-side API
// enter/exit times and the device-side begin/end stamps the kernels write from %globaltimer.
//
// The reference records host enter/exit per RCCL call in its API wrapper
// (rocprofiler-sdk/source/lib/rocprofiler-sdk/rccl/rccl.cpp:145-265) and gets device times from
// a separate kernel-dispatch service that clamps them into the enqueue window
// (rocprofiler-sdk/source/lib/rocprofiler-sdk/tracing/profiling_time.hpp:57-148). Here the
// collective kernel stamps itself, so both live in one record. Device stamps sit in a fixed
// ring; when it is full the tracer drains it (the lossless policy of buffer.hpp:141-166) at the
// cost of one device synchronisation.
#pragma once

#include <stdint.h>

#include <mutex>
#include <string>
#include <vector>

#include "../coll/device.h"
#include "../core/common.h"
#include "b200coll/api_trace.h"

namespace b200 {

class Tracer {
 public:
  Tracer(int rank, int nranks, int cudaDev);
  ~Tracer();
  // Reserve a stamp slot for the next kernel; returns the device pointer to hand to the kernel.
  TraceStamp* begin(int opId, ncclDataType_t dt, uint64_t count, uint64_t bytes);
  void setAlgo(int algo, int ctas);
  void end(bool launchedKernel);
  void drain();  // device stamps -> host records (synchronises the device)
  size_t size();
  uint64_t dropped();
  size_t copyOut(b200collTraceRecordC* out, size_t max);
  void clear();
  bool writeCsv(const std::string& path);
  bool writePerfetto(const std::string& path);

 private:
  static constexpr int kRing = 4096;
  int rank_, nranks_, dev_;
  std::mutex mu_;
  TraceStamp* devRing_ = nullptr;
  int ringUsed_ = 0;
  std::vector<b200collTraceRecordC> recs_;
  std::vector<int> slotOf_;      // ring slot of recs_[i], or -1 once drained / no kernel
  b200collTraceRecordC cur_{};
  int curSlot_ = -1;
  bool open_ = false;
  uint64_t nextCorr_ = 1;
  uint64_t dropped_ = 0;         // records not kept because of TRACE_MAX_RECORDS
};

}  // namespace b200
