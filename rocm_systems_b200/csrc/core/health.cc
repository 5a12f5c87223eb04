// b200smi part 2: watches (sampler thread + per-field ring cache), job statistics, policies and
// the health check — the library half of the reference's RDC daemon
// (rdc/rdc_libs/rdc/src/RdcWatchTableImpl.cc:199-951 watch table and health checks,
//  RdcCacheManagerImpl.cc:36-597 sample cache and job stats, RdcPolicyImpl.cc:59-247 policies).
// Policies only notify; nothing here resets a GPU or changes its settings.
#include <string.h>
#include <time.h>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "b200coll/smi.h"
#include "smi_internal.h"

namespace b200 {
namespace smi {

namespace {

struct Key {
  int dev, field;
  bool operator<(const Key& o) const { return dev != o.dev ? dev < o.dev : field < o.field; }
};
struct Policy { int dev, field; double threshold; int dir; b200smi_policy_cb cb; void* user; bool latched; };
struct Job { bool open = true; std::map<Key, b200smi_stats_t> stats; std::map<Key, double> sum; };

std::mutex gW;
std::condition_variable gCv;
std::thread gThread;
std::atomic<bool> gStop{false};
bool gRunning = false;
std::vector<int> gDevs, gFields;
int gPeriodMs = 1000, gKeep = 600;
std::map<Key, std::deque<b200smi_sample_t>> gCache;
std::vector<Policy> gPolicies;
std::map<std::string, Job> gJobs;

uint64_t nowNs() {
  timespec ts;
  clock_gettime(CLOCK_REALTIME, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + ts.tv_nsec;
}

void sampleOnce() {
  std::vector<int> devs, fields;
  {
    std::lock_guard<std::mutex> lk(gW);
    devs = gDevs;
    fields = gFields;
  }
  for (int d : devs) {
    for (int f : fields) {
      double v = 0;
      if (b200smi_read_field(d, f, &v) != B200SMI_OK) continue;
      b200smi_sample_t s{nowNs(), v};
      std::vector<Policy> fire;
      {
        std::lock_guard<std::mutex> lk(gW);
        auto& q = gCache[Key{d, f}];
        q.push_back(s);
        while ((int)q.size() > gKeep) q.pop_front();
        for (auto& kv : gJobs) {
          Job& j = kv.second;
          if (!j.open) continue;
          b200smi_stats_t& st = j.stats[Key{d, f}];
          if (st.samples == 0) { st.min = st.max = v; }
          if (v < st.min) st.min = v;
          if (v > st.max) st.max = v;
          st.last = v;
          st.samples++;
          j.sum[Key{d, f}] += v;
          st.avg = j.sum[Key{d, f}] / (double)st.samples;
        }
        for (Policy& p : gPolicies) {
          if (p.dev != d || p.field != f) continue;
          const bool hit = p.dir >= 0 ? v > p.threshold : v < p.threshold;
          if (hit && !p.latched) { p.latched = true; fire.push_back(p); }
          if (!hit) p.latched = false;  // re-arm once the value is back inside
        }
      }
      for (const Policy& p : fire) p.cb(d, f, v, p.threshold, p.user);
    }
  }
}

void loop() {
  while (!gStop.load()) {
    sampleOnce();
    std::unique_lock<std::mutex> lk(gW);
    gCv.wait_for(lk, std::chrono::milliseconds(gPeriodMs), [] { return gStop.load(); });
  }
}

}  // namespace

void watchStopLocked() {
  if (!gRunning) return;
  gStop.store(true);
  gCv.notify_all();
  if (gThread.joinable()) gThread.join();
  gRunning = false;
  gStop.store(false);
}

}  // namespace smi
}  // namespace b200

using namespace b200::smi;

extern "C" {

b200smi_status_t b200smi_watch_start(const int* devices, int ndev, const int* fields, int nfields, int periodMs, int keep) {
  if (!ready()) return B200SMI_ERR_NOT_LOADED;
  if (!devices || !fields || ndev <= 0 || nfields <= 0 || periodMs < 1 || keep < 1) return B200SMI_ERR_INVALID;
  watchStopLocked();
  {
    std::lock_guard<std::mutex> lk(gW);
    gDevs.assign(devices, devices + ndev);
    gFields.assign(fields, fields + nfields);
    gPeriodMs = periodMs;
    gKeep = keep;
    gCache.clear();
  }
  gRunning = true;
  gThread = std::thread(loop);
  return B200SMI_OK;
}

b200smi_status_t b200smi_watch_stop(void) {
  watchStopLocked();
  return B200SMI_OK;
}

b200smi_status_t b200smi_watch_latest(int device, int field, b200smi_sample_t* out) {
  if (!out) return B200SMI_ERR_INVALID;
  std::lock_guard<std::mutex> lk(gW);
  auto it = gCache.find(Key{device, field});
  if (it == gCache.end() || it->second.empty()) return B200SMI_ERR_NOT_SUPPORTED;
  *out = it->second.back();
  return B200SMI_OK;
}

b200smi_status_t b200smi_watch_history(int device, int field, b200smi_sample_t* out, int max, int* n) {
  if (!n) return B200SMI_ERR_INVALID;
  std::lock_guard<std::mutex> lk(gW);
  auto it = gCache.find(Key{device, field});
  if (it == gCache.end()) { *n = 0; return B200SMI_OK; }
  int k = 0;
  for (const auto& s : it->second) {
    if (out && k < max) out[k] = s;
    k++;
  }
  *n = k;
  return B200SMI_OK;
}

b200smi_status_t b200smi_job_start(const char* jobId) {
  if (!jobId) return B200SMI_ERR_INVALID;
  std::lock_guard<std::mutex> lk(gW);
  gJobs[jobId] = Job();
  return B200SMI_OK;
}
b200smi_status_t b200smi_job_stop(const char* jobId) {
  if (!jobId) return B200SMI_ERR_INVALID;
  std::lock_guard<std::mutex> lk(gW);
  auto it = gJobs.find(jobId);
  if (it == gJobs.end()) return B200SMI_ERR_INVALID;
  it->second.open = false;
  return B200SMI_OK;
}
b200smi_status_t b200smi_job_stats(const char* jobId, int device, int field, b200smi_stats_t* out) {
  if (!jobId || !out) return B200SMI_ERR_INVALID;
  std::lock_guard<std::mutex> lk(gW);
  auto it = gJobs.find(jobId);
  if (it == gJobs.end()) return B200SMI_ERR_INVALID;
  auto st = it->second.stats.find(Key{device, field});
  if (st == it->second.stats.end()) return B200SMI_ERR_NOT_SUPPORTED;
  *out = st->second;
  return B200SMI_OK;
}

b200smi_status_t b200smi_policy_set(int device, int field, double threshold, int dir, b200smi_policy_cb cb, void* user) {
  if (!cb || field <= 0 || field >= B200SMI_FIELD_COUNT_) return B200SMI_ERR_INVALID;
  std::lock_guard<std::mutex> lk(gW);
  gPolicies.push_back(Policy{device, field, threshold, dir, cb, user, false});
  return B200SMI_OK;
}
b200smi_status_t b200smi_policy_clear(void) {
  std::lock_guard<std::mutex> lk(gW);
  gPolicies.clear();
  return B200SMI_OK;
}

b200smi_status_t b200smi_health(int device, int* level, char* reason, int reasonLen) {
  if (!level) return B200SMI_ERR_INVALID;
  b200smi_device_info_t i;
  b200smi_status_t st = b200smi_device_info(device, &i);
  if (st != B200SMI_OK) return st;
  int lv = 0;
  std::string why;
  auto add = [&](int l, const std::string& s) {
    if (l > lv) lv = l;
    if (!why.empty()) why += "; ";
    why += s;
  };
  if (i.eccUncorrected > 0) add(2, "uncorrected ECC errors: " + std::to_string(i.eccUncorrected));
  if (i.eccCorrected > 0) add(1, "corrected ECC errors: " + std::to_string(i.eccCorrected));
  if (i.nvlinkCount > 0 && i.nvlinkActive < i.nvlinkCount) add(2, "NVLink: " + std::to_string(i.nvlinkActive) + " of " + std::to_string(i.nvlinkCount) + " links up");
  // NVML reason bits: 0x8 hw slowdown, 0x20 sw thermal, 0x40 hw thermal, 0x80 power brake
  if (i.throttleReasons & (0x8ull | 0x40ull | 0x80ull)) add(2, "hardware slowdown active");
  else if (i.throttleReasons & 0x20ull) add(1, "software thermal slowdown active");
  if (i.temperatureC >= 90) add(2, "temperature " + std::to_string(i.temperatureC) + " C");
  else if (i.temperatureC >= 83) add(1, "temperature " + std::to_string(i.temperatureC) + " C");
  *level = lv;
  if (reason && reasonLen > 0) {
    strncpy(reason, why.empty() ? "healthy" : why.c_str(), reasonLen - 1);
    reason[reasonLen - 1] = '\0';
  }
  return B200SMI_OK;
}

}  // extern "C"
