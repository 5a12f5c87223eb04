#include "tracer.h"

#include <string.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <limits>

namespace b200 {

namespace {

__global__ void kReadGlobalTimer(unsigned long long* out) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  *out = t;
}

// What has to be added to a %globaltimer reading of the current GPU to get CLOCK_MONOTONIC nanoseconds. A one-thread
// kernel takes the reading between two reads of the host clock; of several tries the one with the narrowest bracket
// counts and the reading is placed in its middle. 0 when anything fails: device stamps then stay in the GPU's time base.
long long globalTimerOffsetNs() {
  unsigned long long* d = nullptr;
  if (cudaMalloc(&d, sizeof(*d)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  long long best = 0;
  uint64_t bestWidth = ~0ull;
  for (int i = 0; i < 8; i++) {
    cudaDeviceSynchronize();
    const uint64_t t0 = nowNs();
    kReadGlobalTimer<<<1, 1>>>(d);
    unsigned long long g = 0;
    if (cudaMemcpy(&g, d, sizeof(g), cudaMemcpyDeviceToHost) != cudaSuccess || g == 0) {
      (void)cudaGetLastError();
      best = 0;
      break;
    }
    const uint64_t t1 = nowNs();
    if (t1 - t0 < bestWidth) {
      bestWidth = t1 - t0;
      best = (long long)(t0 + (t1 - t0) / 2) - (long long)g;
    }
  }
  cudaFree(d);
  return best;
}

}  // namespace

static const char* kApiNames[] = {
    "ncclAllGather", "ncclAllReduce", "ncclAllToAll", "ncclAllToAllv", "ncclBroadcast", "ncclGather", "ncclReduce",
    "ncclReduceScatter", "ncclScatter", "ncclSend", "ncclRecv", "ncclRedOpCreatePreMulSum", "ncclRedOpDestroy",
    "ncclGroupStart", "ncclGroupEnd", "ncclGetVersion", "ncclGetUniqueId", "ncclCommInitRank", "ncclCommInitAll",
    "ncclCommInitRankConfig", "ncclCommFinalize", "ncclCommDestroy", "ncclCommAbort", "ncclCommSplit",
    "ncclGetErrorString", "ncclGetLastError", "ncclCommGetAsyncError", "ncclCommCount", "ncclCommCuDevice",
    "ncclCommUserRank", "ncclMemAlloc", "ncclMemFree", "mscclLoadAlgo", "mscclRunAlgo", "mscclUnloadAlgo",
    "ncclCommRegister", "ncclCommDeregister"};

Tracer::Tracer(int rank, int nranks, int cudaDev) : rank_(rank), nranks_(nranks), dev_(cudaDev) {
  if (cudaMalloc(&devRing_, sizeof(TraceStamp) * kRing) != cudaSuccess) {
    devRing_ = nullptr;
    (void)cudaGetLastError();
    return;
  }
  std::vector<TraceStamp> init(kRing, TraceStamp{std::numeric_limits<unsigned long long>::max(), 0});
  cudaMemcpy(devRing_, init.data(), sizeof(TraceStamp) * kRing, cudaMemcpyHostToDevice);
}

Tracer::~Tracer() {
  if (devRing_) cudaFree(devRing_);
}

TraceStamp* Tracer::begin(int opId, ncclDataType_t dt, uint64_t count, uint64_t bytes) {
  std::lock_guard<std::mutex> lk(mu_);
  memset(&cur_, 0, sizeof(cur_));
  cur_.correlationId = nextCorr_++;
  cur_.opId = opId;
  cur_.dtype = (int)dt;
  cur_.count = count;
  cur_.bytes = bytes;
  cur_.hostBeginNs = nowNs();
  open_ = true;
  curSlot_ = -1;
  if (!devRing_) return nullptr;
  if (ringUsed_ == kRing) {
    mu_.unlock();
    drain();
    mu_.lock();
  }
  curSlot_ = ringUsed_++;
  return devRing_ + curSlot_;
}

void Tracer::setAlgo(int algo, int ctas) {
  std::lock_guard<std::mutex> lk(mu_);
  cur_.algo = algo;
  cur_.ctas = ctas;
}

void Tracer::end(bool launchedKernel) {
  std::lock_guard<std::mutex> lk(mu_);
  if (!open_) return;
  open_ = false;
  cur_.hostEndNs = nowNs();
  if (!launchedKernel && curSlot_ >= 0 && curSlot_ == ringUsed_ - 1) {
    ringUsed_--;  // give the untouched slot back
    curSlot_ = -1;
  }
  // Lossless by default; with a limit the first records are kept and later ones only counted (the two buffer policies of the
  // reference's record buffers, rocprofiler-sdk source/lib/rocprofiler-sdk/buffer.hpp:141-166). A dropped record's ring slot
  // is simply never read back.
  const long long limit = Flags::get().traceMaxRecords;
  if (limit > 0 && (long long)recs_.size() >= limit) {
    dropped_++;
    return;
  }
  recs_.push_back(cur_);
  slotOf_.push_back(launchedKernel ? curSlot_ : -1);
}

uint64_t Tracer::dropped() {
  std::lock_guard<std::mutex> lk(mu_);
  return dropped_;
}

void Tracer::drain() {
  std::lock_guard<std::mutex> lk(mu_);
  if (!devRing_ || ringUsed_ == 0) return;
  int prev = -1;
  cudaGetDevice(&prev);
  if (prev != dev_) cudaSetDevice(dev_);
  cudaDeviceSynchronize();
  std::vector<TraceStamp> host(ringUsed_);
  cudaMemcpy(host.data(), devRing_, sizeof(TraceStamp) * ringUsed_, cudaMemcpyDeviceToHost);
  const long long offset = globalTimerOffsetNs();
  const uint64_t now = nowNs();
  for (size_t i = 0; i < recs_.size(); i++) {
    int s = slotOf_[i];
    if (s < 0 || s >= ringUsed_) continue;
    unsigned long long b = host[s].begin, e = host[s].end;
    if (b == std::numeric_limits<unsigned long long>::max() || e == 0) { b = 0; e = 0; }
    if (e < b) std::swap(b, e);  // same repair the reference applies to swapped device stamps
    if (e != 0) {
      // Into the host's clock, then the reference's two shifts against clock skew, which keep the duration
      // (rocprofiler-sdk tracing/profiling_time.hpp:137-145): the interval ends no later than now and starts no
      // earlier than the call that enqueued it.
      long long B = (long long)b + offset, E = (long long)e + offset;
      if (E > (long long)now) { B -= E - (long long)now; E = (long long)now; }
      if (B < (long long)recs_[i].hostBeginNs) { E += (long long)recs_[i].hostBeginNs - B; B = (long long)recs_[i].hostBeginNs; }
      b = (unsigned long long)B;
      e = (unsigned long long)E;
    }
    recs_[i].devBeginNs = b;
    recs_[i].devEndNs = e;
    slotOf_[i] = -1;
  }
  std::vector<TraceStamp> init(ringUsed_, TraceStamp{std::numeric_limits<unsigned long long>::max(), 0});
  cudaMemcpy(devRing_, init.data(), sizeof(TraceStamp) * ringUsed_, cudaMemcpyHostToDevice);
  ringUsed_ = 0;
  if (prev != dev_ && prev >= 0) cudaSetDevice(prev);
}

size_t Tracer::size() {
  std::lock_guard<std::mutex> lk(mu_);
  return recs_.size();
}

size_t Tracer::copyOut(b200collTraceRecordC* out, size_t max) {
  std::lock_guard<std::mutex> lk(mu_);
  size_t n = recs_.size() < max ? recs_.size() : max;
  if (out && n) memcpy(out, recs_.data(), n * sizeof(b200collTraceRecordC));
  return recs_.size();
}

void Tracer::clear() {
  drain();
  std::lock_guard<std::mutex> lk(mu_);
  recs_.clear();
  slotOf_.clear();
}

// Columns: the reference's RCCL trace CSV (Domain, Function, Process_Id, Thread_Id,
// Correlation_Id, Start_Timestamp, End_Timestamp; rocprofiler-sdk/source/docs/data/rccl_trace.csv)
// followed by what this tracer adds.
bool Tracer::writeCsv(const std::string& path) {
  std::lock_guard<std::mutex> lk(mu_);
  FILE* f = fopen(path.c_str(), "w");
  if (!f) return false;
  fprintf(f, "\"Domain\",\"Function\",\"Process_Id\",\"Thread_Id\",\"Correlation_Id\",\"Start_Timestamp\",\"End_Timestamp\","
             "\"Rank\",\"Count\",\"Dtype\",\"Bytes\",\"Algo\",\"Ctas\",\"Device_Start\",\"Device_End\",\"Device_Us\",\"AlgBw_GBps\"\n");
  long tid = syscall(SYS_gettid);
  for (const auto& r : recs_) {
    double us = r.devEndNs > r.devBeginNs ? (r.devEndNs - r.devBeginNs) / 1e3 : 0.0;
    double bw = us > 0 ? (double)r.bytes / us / 1e3 : 0.0;
    fprintf(f, "\"B200COLL_API\",\"%s\",%d,%ld,%llu,%llu,%llu,%d,%llu,\"%s\",%llu,%d,%d,%llu,%llu,%.3f,%.3f\n", b200collApiName(r.opId), (int)getpid(), tid,
            (unsigned long long)r.correlationId, (unsigned long long)r.hostBeginNs, (unsigned long long)r.hostEndNs, rank_,
            (unsigned long long)r.count, dtypeName((ncclDataType_t)r.dtype), (unsigned long long)r.bytes, r.algo, r.ctas,
            (unsigned long long)r.devBeginNs, (unsigned long long)r.devEndNs, us, bw);
  }
  fclose(f);
  return true;
}

// Chrome/Perfetto JSON trace: host API slices on one track, device slices on another, and a
// byte counter per collective (the "Comm Send/Recv" counter tracks of
// rocprofiler-systems/source/lib/rocprof-sys/library/rocprofiler-sdk/rccl.cpp:105-180).
bool Tracer::writePerfetto(const std::string& path) {
  std::lock_guard<std::mutex> lk(mu_);
  FILE* f = fopen(path.c_str(), "w");
  if (!f) return false;
  fprintf(f, "{\"traceEvents\":[\n");
  bool first = true;
  uint64_t total = 0;
  for (const auto& r : recs_) {
    const char* name = b200collApiName(r.opId);
    fprintf(f, "%s{\"name\":\"%s\",\"cat\":\"b200coll_api\",\"ph\":\"X\",\"pid\":%d,\"tid\":0,\"ts\":%.3f,\"dur\":%.3f,\"args\":{\"count\":%llu,\"bytes\":%llu,\"corr\":%llu}}",
            first ? "" : ",\n", name, rank_, r.hostBeginNs / 1e3, (r.hostEndNs - r.hostBeginNs) / 1e3, (unsigned long long)r.count,
            (unsigned long long)r.bytes, (unsigned long long)r.correlationId);
    first = false;
    if (r.devEndNs > r.devBeginNs)
      fprintf(f, ",\n{\"name\":\"%s\",\"cat\":\"b200coll_device\",\"ph\":\"X\",\"pid\":%d,\"tid\":1,\"ts\":%.3f,\"dur\":%.3f,\"args\":{\"corr\":%llu}}", name, rank_,
              r.devBeginNs / 1e3, (r.devEndNs - r.devBeginNs) / 1e3, (unsigned long long)r.correlationId);
    total += r.bytes;
    fprintf(f, ",\n{\"name\":\"Comm Bytes\",\"ph\":\"C\",\"pid\":%d,\"ts\":%.3f,\"args\":{\"bytes\":%llu}}", rank_, r.hostBeginNs / 1e3, (unsigned long long)total);
  }
  fprintf(f, "\n]}\n");
  fclose(f);
  return true;
}

}  // namespace b200

extern "C" const char* b200collApiName(int apiId) {
  if (apiId < 0 || apiId >= B200COLL_API_ID_LAST) return "unknown";
  return b200::kApiNames[apiId];
}
