// b200smi part 1: NVML loading, device readings and the link (topology) table.
//
// The reference discovers topology from sysfs (libhsakmt/src/topology.c:56-59, 1634-1931) and
// exposes it through rocm-smi (rocm-smi-lib/src/rocm_smi.cc:4665-4910). On a B200 box every pair of
// GPUs is one NVSwitch hop apart at full link bandwidth, so the table is uniform; it is still
// derived from what NVML and the CUDA runtime report (links up, peer access, native atomics).
#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <nvml.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include <mutex>
#include <utility>

#include "b200coll/smi.h"
#include "mem.h"
#include "smi_internal.h"

namespace b200 {
namespace smi {

static std::mutex gMu;
static int gRef = 0;
static void* gLib = nullptr;
NvmlFns gN;

template <typename F> static bool sym(const char* name, F* out, bool required = true) {
  *out = reinterpret_cast<F>(dlsym(gLib, name));
  return *out != nullptr || !required;
}

static bool loadNvml() {
  const char* override = getenv("B200SMI_NVML_LIBRARY");
  const char* names[] = {override, "libnvidia-ml.so.1", "libnvidia-ml.so"};
  for (const char* n : names) {
    if (!n || !*n) continue;
    gLib = dlopen(n, RTLD_NOW | RTLD_LOCAL);
    if (gLib) break;
  }
  if (!gLib) return false;
  bool ok = true;
  ok &= sym("nvmlInit_v2", &gN.init);
  ok &= sym("nvmlShutdown", &gN.shutdown);
  ok &= sym("nvmlDeviceGetCount_v2", &gN.count);
  ok &= sym("nvmlDeviceGetHandleByIndex_v2", &gN.handle);
  ok &= sym("nvmlDeviceGetName", &gN.name);
  sym("nvmlDeviceGetUUID", &gN.uuid, false);
  sym("nvmlDeviceGetPciInfo_v3", &gN.pci, false);
  sym("nvmlDeviceGetClockInfo", &gN.clock, false);
  sym("nvmlDeviceGetMaxClockInfo", &gN.maxClock, false);
  sym("nvmlDeviceGetPowerUsage", &gN.power, false);
  sym("nvmlDeviceGetEnforcedPowerLimit", &gN.powerLimit, false);
  sym("nvmlDeviceGetTemperature", &gN.temp, false);
  sym("nvmlDeviceGetMemoryInfo", &gN.mem, false);
  sym("nvmlDeviceGetTotalEccErrors", &gN.ecc, false);
  sym("nvmlDeviceGetCurrentClocksEventReasons", &gN.reasons, false);
  if (!gN.reasons) sym("nvmlDeviceGetCurrentClocksThrottleReasons", &gN.reasons, false);
  sym("nvmlDeviceGetUtilizationRates", &gN.util, false);
  sym("nvmlDeviceGetNvLinkState", &gN.nvlinkState, false);
  sym("nvmlDeviceGetNvLinkRemotePciInfo_v2", &gN.nvlinkRemote, false);
  sym("nvmlDeviceSetPowerManagementLimit", &gN.setPowerLimit, false);
  sym("nvmlSystemGetDriverVersion", &gN.driverVersion, false);
  sym("nvmlDeviceGetComputeRunningProcesses_v3", &gN.processes, false);
  sym("nvmlDeviceGetNvLinkErrorCounter", &gN.nvlinkError, false);
  sym("nvmlDeviceGetCurrPcieLinkGeneration", &gN.pcieGen, false);
  sym("nvmlDeviceGetCurrPcieLinkWidth", &gN.pcieWidth, false);
  sym("nvmlDeviceGetComputeMode", &gN.computeMode, false);
  sym("nvmlDeviceGetPersistenceMode", &gN.persistence, false);
  sym("nvmlDeviceGetMigMode", &gN.migMode, false);
  sym("nvmlDeviceGetEccMode", &gN.eccMode, false);
  sym("nvmlEventSetCreate", &gN.eventSetCreate, false);
  sym("nvmlEventSetFree", &gN.eventSetFree, false);
  sym("nvmlDeviceGetSupportedEventTypes", &gN.supportedEvents, false);
  sym("nvmlDeviceRegisterEvents", &gN.registerEvents, false);
  sym("nvmlEventSetWait_v2", &gN.eventSetWait, false);
  sym("nvmlDeviceGetCpuAffinity", &gN.cpuAffinity, false);
  sym("nvmlDeviceGetNumaNodeId", &gN.numaNode, false);
  sym("nvmlDeviceGetSerial", &gN.serial, false);
  sym("nvmlDeviceGetBoardPartNumber", &gN.partNumber, false);
  sym("nvmlDeviceGetVbiosVersion", &gN.vbios, false);
  sym("nvmlDeviceGetInforomImageVersion", &gN.inforomImage, false);
  sym("nvmlDeviceGetPerformanceState", &gN.pstate, false);
  sym("nvmlDeviceGetPowerManagementLimitConstraints", &gN.powerConstraints, false);
  sym("nvmlDeviceGetTotalEnergyConsumption", &gN.energy, false);
  sym("nvmlDeviceGetRemappedRows", &gN.remappedRows, false);
  sym("nvmlDeviceSetGpuLockedClocks", &gN.setLockedClocks, false);
  sym("nvmlDeviceResetGpuLockedClocks", &gN.resetLockedClocks, false);
  sym("nvmlGpmQueryDeviceSupport", &gN.gpmSupport, false);
  sym("nvmlGpmSampleAlloc", &gN.gpmSampleAlloc, false);
  sym("nvmlGpmSampleFree", &gN.gpmSampleFree, false);
  sym("nvmlGpmSampleGet", &gN.gpmSampleGet, false);
  sym("nvmlGpmMetricsGet", &gN.gpmMetricsGet, false);
  if (!ok) {
    dlclose(gLib);
    gLib = nullptr;
  }
  return ok;
}

bool ready() { return gRef > 0; }

b200smi_status_t deviceHandle(int device, nvmlDevice_t* h) {
  if (!ready()) return B200SMI_ERR_NOT_LOADED;
  unsigned n = 0;
  if (gN.count(&n) != NVML_SUCCESS) return B200SMI_ERR_NVML;
  if (device < 0 || device >= (int)n) return B200SMI_ERR_INVALID;
  return gN.handle((unsigned)device, h) == NVML_SUCCESS ? B200SMI_OK : B200SMI_ERR_NVML;
}

static void countLinks(nvmlDevice_t h, uint32_t* total, uint32_t* active) {
  *total = 0;
  *active = 0;
  if (!gN.nvlinkState) return;
  for (unsigned l = 0; l < NVML_NVLINK_MAX_LINKS; l++) {
    nvmlEnableState_t st;
    nvmlReturn_t r = gN.nvlinkState(h, l, &st);
    if (r != NVML_SUCCESS) continue;  // link index not present on this part
    (*total)++;
    if (st == NVML_FEATURE_ENABLED) (*active)++;
  }
}

}  // namespace smi
}  // namespace b200

namespace {
struct ActivityState {
  nvmlGpmSample_t prev = nullptr, cur = nullptr;
  uint64_t prevNs = 0;          // when `prev` was taken; 0: none yet
  uint64_t resultNs = 0;
  b200smi_activity_t result{};
  int supported = -1;           // -1 not asked yet
};
std::mutex gActMu;
ActivityState gAct[64];

uint64_t monoNs() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}
}  // namespace

namespace b200 {
namespace smi {
void activityReset() {  // at the last shutdown: the samples belong to the library that is about to be closed
  std::lock_guard<std::mutex> lk(gActMu);
  for (auto& a : gAct) {
    if (gN.gpmSampleFree) {
      if (a.prev) gN.gpmSampleFree(a.prev);
      if (a.cur) gN.gpmSampleFree(a.cur);
    }
    a = ActivityState{};
  }
}
}  // namespace smi
}  // namespace b200

using namespace b200::smi;

extern "C" {

b200smi_status_t b200smi_init(void) {
  std::lock_guard<std::mutex> lk(gMu);
  if (gRef > 0) { gRef++; return B200SMI_OK; }
  if (!gLib && !loadNvml()) return B200SMI_ERR_NOT_LOADED;
  if (gN.init() != NVML_SUCCESS) return B200SMI_ERR_NVML;
  gRef = 1;
  return B200SMI_OK;
}

b200smi_status_t b200smi_shutdown(void) {
  std::lock_guard<std::mutex> lk(gMu);
  if (gRef == 0) return B200SMI_ERR_NOT_LOADED;
  if (--gRef == 0) {
    watchStopLocked();
    activityReset();
    gN.shutdown();
  }
  return B200SMI_OK;
}

const char* b200smi_status_string(b200smi_status_t s) {
  switch (s) {
    case B200SMI_OK: return "ok";
    case B200SMI_ERR_NOT_LOADED: return "NVML is not loaded (no driver on this machine, or b200smi_init was not called)";
    case B200SMI_ERR_INVALID: return "invalid argument";
    case B200SMI_ERR_NOT_SUPPORTED: return "not supported by this device or driver";
    case B200SMI_ERR_PERMISSION: return "changing GPU settings is disabled (needs B200SMI_ALLOW_SET=1 and allow=1)";
    case B200SMI_ERR_TIMEOUT: return "nothing happened within the time given";
    default: return "NVML call failed";
  }
}

b200smi_status_t b200smi_device_count(int* count) {
  if (!count) return B200SMI_ERR_INVALID;
  if (!ready()) return B200SMI_ERR_NOT_LOADED;
  unsigned n = 0;
  if (gN.count(&n) != NVML_SUCCESS) return B200SMI_ERR_NVML;
  *count = (int)n;
  return B200SMI_OK;
}

b200smi_status_t b200smi_device_info(int device, b200smi_device_info_t* info) {
  if (!info) return B200SMI_ERR_INVALID;
  nvmlDevice_t h;
  b200smi_status_t st = deviceHandle(device, &h);
  if (st != B200SMI_OK) return st;
  memset(info, 0, sizeof(*info));
  gN.name(h, info->name, sizeof(info->name));
  if (gN.uuid) gN.uuid(h, info->uuid, sizeof(info->uuid));
  if (gN.pci) {
    nvmlPciInfo_t p;
    if (gN.pci(h, &p) == NVML_SUCCESS) strncpy(info->busId, p.busId, sizeof(info->busId) - 1);
  }
  if (gN.clock) {
    gN.clock(h, NVML_CLOCK_SM, &info->smClockMhz);
    gN.clock(h, NVML_CLOCK_MEM, &info->memClockMhz);
  }
  if (gN.maxClock) {
    gN.maxClock(h, NVML_CLOCK_SM, &info->smClockMaxMhz);
    gN.maxClock(h, NVML_CLOCK_MEM, &info->memClockMaxMhz);
  }
  if (gN.power) gN.power(h, &info->powerMilliwatt);
  if (gN.powerLimit) gN.powerLimit(h, &info->powerLimitMilliwatt);
  if (gN.temp) gN.temp(h, NVML_TEMPERATURE_GPU, &info->temperatureC);
  if (gN.mem) {
    nvmlMemory_t m;
    if (gN.mem(h, &m) == NVML_SUCCESS) { info->memTotalBytes = m.total; info->memUsedBytes = m.used; }
  }
  if (gN.ecc) {
    unsigned long long c = 0;
    if (gN.ecc(h, NVML_MEMORY_ERROR_TYPE_CORRECTED, NVML_VOLATILE_ECC, &c) == NVML_SUCCESS) info->eccCorrected = c;
    if (gN.ecc(h, NVML_MEMORY_ERROR_TYPE_UNCORRECTED, NVML_VOLATILE_ECC, &c) == NVML_SUCCESS) info->eccUncorrected = c;
  }
  if (gN.reasons) {
    unsigned long long r = 0;
    if (gN.reasons(h, &r) == NVML_SUCCESS) info->throttleReasons = r;
  }
  if (gN.util) {
    nvmlUtilization_t u;
    if (gN.util(h, &u) == NVML_SUCCESS) { info->gpuUtilPct = u.gpu; info->memUtilPct = u.memory; }
  }
  countLinks(h, &info->nvlinkCount, &info->nvlinkActive);
  b200::MemCaps caps;
  if (b200::queryMemCaps(device, &caps) == ncclSuccess) info->multicastCapable = caps.multicast ? 1 : 0;
  return B200SMI_OK;
}

// ---- activity from performance-monitoring samples --------------------------------------------------------------------
// Two samples bracket an interval; the driver turns the pair into percentages and rates. Per device the previous sample
// is kept, so a periodic reader (the watch thread, a monitor loop) pays one sample per period and gets the activity of
// exactly that period. This is what the reference's telemetry gets from its profiler plug-in
// (rdc/rdc_libs/rdc_modules/rdc_rocp/RdcRocpBase.cpp: occupancy, active cycles, FLOP rates as watchable fields),
// without programming counters: the samples come from the driver's always-on monitoring block.
b200smi_status_t b200smi_activity(int device, b200smi_activity_t* out) {
  if (!out) return B200SMI_ERR_INVALID;
  nvmlDevice_t h;
  b200smi_status_t st = deviceHandle(device, &h);
  if (st != B200SMI_OK) return st;
  if (device >= 64) return B200SMI_ERR_INVALID;
  if (!gN.gpmSampleAlloc || !gN.gpmSampleGet || !gN.gpmMetricsGet) return B200SMI_ERR_NOT_SUPPORTED;
  std::lock_guard<std::mutex> lk(gActMu);
  ActivityState& a = gAct[device];
  if (a.supported < 0) {
    a.supported = 1;
    if (gN.gpmSupport) {
      nvmlGpmSupport_t sup;
      memset(&sup, 0, sizeof(sup));
      sup.version = NVML_GPM_SUPPORT_VERSION;
      if (gN.gpmSupport(h, &sup) != NVML_SUCCESS || !sup.isSupportedDevice) a.supported = 0;
    }
  }
  if (!a.supported) return B200SMI_ERR_NOT_SUPPORTED;
  uint64_t now = monoNs();
  if (a.resultNs && now - a.resultNs < 50000000ull) {  // several fields read in a row share one interval
    *out = a.result;
    return B200SMI_OK;
  }
  if (!a.prev && gN.gpmSampleAlloc(&a.prev) != NVML_SUCCESS) return B200SMI_ERR_NVML;
  if (!a.cur && gN.gpmSampleAlloc(&a.cur) != NVML_SUCCESS) return B200SMI_ERR_NVML;
  if (!a.prevNs || now - a.prevNs > 5000000000ull) {
    if (gN.gpmSampleGet(h, a.prev) != NVML_SUCCESS) return B200SMI_ERR_NVML;
    a.prevNs = now;
    timespec nap{0, 100000000};
    nanosleep(&nap, nullptr);
    now = monoNs();
  }
  if (gN.gpmSampleGet(h, a.cur) != NVML_SUCCESS) return B200SMI_ERR_NVML;
  static const unsigned ids[] = {NVML_GPM_METRIC_SM_UTIL, NVML_GPM_METRIC_SM_OCCUPANCY, NVML_GPM_METRIC_ANY_TENSOR_UTIL, NVML_GPM_METRIC_DRAM_BW_UTIL,
                                 NVML_GPM_METRIC_FP64_UTIL, NVML_GPM_METRIC_FP32_UTIL, NVML_GPM_METRIC_FP16_UTIL, NVML_GPM_METRIC_PCIE_TX_PER_SEC,
                                 NVML_GPM_METRIC_PCIE_RX_PER_SEC, NVML_GPM_METRIC_NVLINK_TOTAL_TX_PER_SEC, NVML_GPM_METRIC_NVLINK_TOTAL_RX_PER_SEC};
  constexpr unsigned n = sizeof(ids) / sizeof(ids[0]);
  static nvmlGpmMetricsGet_t req;  // large (one slot per metric the driver knows): not on the stack; gActMu is held
  memset(&req, 0, sizeof(req));
  req.version = NVML_GPM_METRICS_GET_VERSION;
  req.numMetrics = n;
  req.sample1 = a.prev;
  req.sample2 = a.cur;
  for (unsigned i = 0; i < n; i++) req.metrics[i].metricId = ids[i];
  if (gN.gpmMetricsGet(&req) != NVML_SUCCESS) return B200SMI_ERR_NVML;
  double v[n];
  for (unsigned i = 0; i < n; i++) v[i] = req.metrics[i].nvmlReturn == NVML_SUCCESS ? req.metrics[i].value : -1.0;
  a.result = b200smi_activity_t{(now - a.prevNs) / 1e6, v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], v[8], v[9], v[10]};
  a.resultNs = now;
  std::swap(a.prev, a.cur);
  a.prevNs = now;
  *out = a.result;
  return B200SMI_OK;
}

b200smi_status_t b200smi_read_field(int device, int field, double* value) {
  if (!value) return B200SMI_ERR_INVALID;
  if (field >= B200SMI_FIELD_SM_ACTIVE && field <= B200SMI_FIELD_NVLINK_RX_MIBS) {
    b200smi_activity_t act;
    b200smi_status_t ast = b200smi_activity(device, &act);
    if (ast != B200SMI_OK) return ast;
    const double vals[] = {act.smActivePct, act.smOccupancyPct, act.tensorActivePct, act.dramActivePct, act.fp64ActivePct, act.fp32ActivePct,
                           act.fp16ActivePct, act.pcieTxMiBs, act.pcieRxMiBs, act.nvlinkTxMiBs, act.nvlinkRxMiBs};
    *value = vals[field - B200SMI_FIELD_SM_ACTIVE];
    return *value < 0 ? B200SMI_ERR_NOT_SUPPORTED : B200SMI_OK;
  }
  b200smi_device_info_t i;
  b200smi_status_t st = b200smi_device_info(device, &i);
  if (st != B200SMI_OK) return st;
  switch (field) {
    case B200SMI_FIELD_SM_CLOCK: *value = i.smClockMhz; break;
    case B200SMI_FIELD_MEM_CLOCK: *value = i.memClockMhz; break;
    case B200SMI_FIELD_POWER: *value = i.powerMilliwatt / 1000.0; break;
    case B200SMI_FIELD_TEMP: *value = i.temperatureC; break;
    case B200SMI_FIELD_MEM_USED: *value = (double)i.memUsedBytes; break;
    case B200SMI_FIELD_GPU_UTIL: *value = i.gpuUtilPct; break;
    case B200SMI_FIELD_MEM_UTIL: *value = i.memUtilPct; break;
    case B200SMI_FIELD_ECC_CORRECTED: *value = (double)i.eccCorrected; break;
    case B200SMI_FIELD_ECC_UNCORRECTED: *value = (double)i.eccUncorrected; break;
    case B200SMI_FIELD_THROTTLE_REASONS: *value = (double)i.throttleReasons; break;
    case B200SMI_FIELD_NVLINK_ACTIVE: *value = i.nvlinkActive; break;
    default: return B200SMI_ERR_INVALID;
  }
  return B200SMI_OK;
}

b200smi_status_t b200smi_link(int from, int to, b200smi_link_t* link) {
  if (!link) return B200SMI_ERR_INVALID;
  nvmlDevice_t hf, ht;
  b200smi_status_t st = deviceHandle(from, &hf);
  if (st != B200SMI_OK) return st;
  st = deviceHandle(to, &ht);
  if (st != B200SMI_OK) return st;
  memset(link, 0, sizeof(*link));
  link->perfRank = -1;
  if (from == to) {
    link->type = B200SMI_LINK_SELF;
    link->p2pAccessible = link->atomics32 = link->atomics64 = link->coherent = 1;
    return B200SMI_OK;
  }
  uint32_t total = 0, active = 0, total2 = 0, active2 = 0;
  countLinks(hf, &total, &active);
  countLinks(ht, &total2, &active2);
  const uint32_t up = active < active2 ? active : active2;
  if (up > 0) {
    // Every link of a B200 goes to the NVSwitch fabric, so the pair is one switch hop apart and
    // can use all links that are up on both ends: 50 GB/s per direction per NVLink-5 link.
    link->type = B200SMI_LINK_NVLINK;
    link->hops = 1;
    link->weight = 15;
    link->nvlinks = up;
    link->minBandwidthMBps = 50000ull;
    link->maxBandwidthMBps = 50000ull * up;
  } else {
    link->type = B200SMI_LINK_PCIE;
    link->hops = 2;
    link->weight = 40;
    link->minBandwidthMBps = link->maxBandwidthMBps = 64000ull;
  }
  int can = 0, atom = 0, rank = -1;
  if (cudaDeviceCanAccessPeer(&can, from, to) == cudaSuccess) {
    link->p2pAccessible = can;
    if (cudaDeviceGetP2PAttribute(&atom, cudaDevP2PAttrNativeAtomicSupported, from, to) == cudaSuccess) link->atomics32 = link->atomics64 = atom;
    if (cudaDeviceGetP2PAttribute(&rank, cudaDevP2PAttrPerformanceRank, from, to) == cudaSuccess) link->perfRank = rank;
  } else {
    (void)cudaGetLastError();
    // No CUDA runtime view (e.g. a management-only process): NVLink peers are addressable and atomic-capable.
    link->p2pAccessible = link->type == B200SMI_LINK_NVLINK;
    link->atomics32 = link->atomics64 = link->type == B200SMI_LINK_NVLINK;
  }
  link->coherent = link->p2pAccessible;
  return B200SMI_OK;
}

b200smi_status_t b200smi_set_power_limit(int device, uint32_t milliwatt, int allow) {
  const char* env = getenv("B200SMI_ALLOW_SET");
  if (!allow || !env || strcmp(env, "1") != 0) return B200SMI_ERR_PERMISSION;
  nvmlDevice_t h;
  b200smi_status_t st = deviceHandle(device, &h);
  if (st != B200SMI_OK) return st;
  if (!gN.setPowerLimit) return B200SMI_ERR_NOT_SUPPORTED;
  return gN.setPowerLimit(h, milliwatt) == NVML_SUCCESS ? B200SMI_OK : B200SMI_ERR_NVML;
}

static bool settersAllowed(int allow) {
  const char* env = getenv("B200SMI_ALLOW_SET");
  return allow && env && strcmp(env, "1") == 0;
}

b200smi_status_t b200smi_set_locked_clocks(int device, uint32_t minMhz, uint32_t maxMhz, int allow) {
  if (!settersAllowed(allow)) return B200SMI_ERR_PERMISSION;
  if (minMhz == 0 || maxMhz < minMhz) return B200SMI_ERR_INVALID;
  nvmlDevice_t h;
  b200smi_status_t st = deviceHandle(device, &h);
  if (st != B200SMI_OK) return st;
  if (!gN.setLockedClocks) return B200SMI_ERR_NOT_SUPPORTED;
  return gN.setLockedClocks(h, minMhz, maxMhz) == NVML_SUCCESS ? B200SMI_OK : B200SMI_ERR_NVML;
}

b200smi_status_t b200smi_reset_locked_clocks(int device, int allow) {
  if (!settersAllowed(allow)) return B200SMI_ERR_PERMISSION;
  nvmlDevice_t h;
  b200smi_status_t st = deviceHandle(device, &h);
  if (st != B200SMI_OK) return st;
  if (!gN.resetLockedClocks) return B200SMI_ERR_NOT_SUPPORTED;
  return gN.resetLockedClocks(h) == NVML_SUCCESS ? B200SMI_OK : B200SMI_ERR_NVML;
}

b200smi_status_t b200smi_cpu_affinity(int device, uint64_t* mask, int words, int* numaNode) {
  if (!mask || words <= 0 || words > 64) return B200SMI_ERR_INVALID;
  nvmlDevice_t h;
  b200smi_status_t st = deviceHandle(device, &h);
  if (st != B200SMI_OK) return st;
  if (!gN.cpuAffinity) return B200SMI_ERR_NOT_SUPPORTED;
  static_assert(sizeof(unsigned long) == sizeof(uint64_t), "one NVML affinity word is 64 bits here");
  memset(mask, 0, sizeof(uint64_t) * words);
  if (gN.cpuAffinity(h, (unsigned)words, (unsigned long*)mask) != NVML_SUCCESS) return B200SMI_ERR_NVML;
  if (numaNode) {
    unsigned int node = 0;
    *numaNode = (gN.numaNode && gN.numaNode(h, &node) == NVML_SUCCESS) ? (int)node : -1;
  }
  return B200SMI_OK;
}

b200smi_status_t b200smi_identity(int device, b200smi_identity_t* out) {
  if (!out) return B200SMI_ERR_INVALID;
  nvmlDevice_t h;
  b200smi_status_t st = deviceHandle(device, &h);
  if (st != B200SMI_OK) return st;
  memset(out, 0, sizeof(*out));
  out->performanceState = -1;
  out->powerLimitMinMilliwatt = out->powerLimitMaxMilliwatt = out->energyMillijoule = -1;
  out->remappedCorrectable = out->remappedUncorrectable = out->remapPending = out->remapFailed = -1;
  if (gN.serial && gN.serial(h, out->serial, sizeof(out->serial)) != NVML_SUCCESS) out->serial[0] = 0;
  if (gN.partNumber && gN.partNumber(h, out->partNumber, sizeof(out->partNumber)) != NVML_SUCCESS) out->partNumber[0] = 0;
  if (gN.vbios && gN.vbios(h, out->vbios, sizeof(out->vbios)) != NVML_SUCCESS) out->vbios[0] = 0;
  if (gN.inforomImage && gN.inforomImage(h, out->inforomImage, sizeof(out->inforomImage)) != NVML_SUCCESS) out->inforomImage[0] = 0;
  nvmlPstates_t ps;
  if (gN.pstate && gN.pstate(h, &ps) == NVML_SUCCESS && ps != NVML_PSTATE_UNKNOWN) out->performanceState = (int)ps;
  unsigned int lo = 0, hi = 0;
  if (gN.powerConstraints && gN.powerConstraints(h, &lo, &hi) == NVML_SUCCESS) {
    out->powerLimitMinMilliwatt = lo;
    out->powerLimitMaxMilliwatt = hi;
  }
  unsigned long long mj = 0;
  if (gN.energy && gN.energy(h, &mj) == NVML_SUCCESS) out->energyMillijoule = (int64_t)mj;
  unsigned int corr = 0, unc = 0, pending = 0, failed = 0;
  if (gN.remappedRows && gN.remappedRows(h, &corr, &unc, &pending, &failed) == NVML_SUCCESS) {
    out->remappedCorrectable = (int)corr;
    out->remappedUncorrectable = (int)unc;
    out->remapPending = (int)pending;
    out->remapFailed = (int)failed;
  }
  return B200SMI_OK;
}

}  // extern "C"

// ---- driver, processes, link errors, PCIe ------------------------------------------------------
extern "C" {

b200smi_status_t b200smi_driver_version(char* buf, int len) {
  using namespace b200::smi;
  if (!buf || len < 2) return B200SMI_ERR_INVALID;
  if (!ready()) return B200SMI_ERR_NOT_LOADED;
  if (!gN.driverVersion) return B200SMI_ERR_NOT_SUPPORTED;
  return gN.driverVersion(buf, (unsigned)len) == NVML_SUCCESS ? B200SMI_OK : B200SMI_ERR_NVML;
}

b200smi_status_t b200smi_processes(int device, b200smi_process_t* out, int max, int* n) {
  using namespace b200::smi;
  if (!n || max < 0 || (max > 0 && !out)) return B200SMI_ERR_INVALID;
  nvmlDevice_t h;
  b200smi_status_t st = deviceHandle(device, &h);
  if (st != B200SMI_OK) return st;
  if (!gN.processes) return B200SMI_ERR_NOT_SUPPORTED;
  nvmlProcessInfo_t infos[256];
  unsigned int count = 256;
  nvmlReturn_t r = gN.processes(h, &count, infos);
  if (r != NVML_SUCCESS && r != NVML_ERROR_INSUFFICIENT_SIZE) return B200SMI_ERR_NVML;
  if (count > 256) count = 256;
  *n = (int)count;
  for (unsigned i = 0; i < count && (int)i < max; i++) {
    out[i].pid = infos[i].pid;
    out[i].usedMemoryBytes = infos[i].usedGpuMemory;
    out[i].name[0] = 0;
    char path[64];
    snprintf(path, sizeof(path), "/proc/%u/comm", infos[i].pid);
    if (FILE* f = fopen(path, "r")) {
      if (fgets(out[i].name, sizeof(out[i].name), f)) {
        size_t l = strlen(out[i].name);
        if (l && out[i].name[l - 1] == '\n') out[i].name[l - 1] = 0;
      }
      fclose(f);
    }
  }
  return B200SMI_OK;
}

b200smi_status_t b200smi_nvlink_errors(int device, b200smi_nvlink_errors_t* out) {
  using namespace b200::smi;
  if (!out) return B200SMI_ERR_INVALID;
  nvmlDevice_t h;
  b200smi_status_t st = deviceHandle(device, &h);
  if (st != B200SMI_OK) return st;
  if (!gN.nvlinkError) return B200SMI_ERR_NOT_SUPPORTED;
  memset(out, 0, sizeof(*out));
  for (unsigned link = 0; link < NVML_NVLINK_MAX_LINKS; link++) {
    unsigned long long v = 0;
    if (gN.nvlinkError(h, link, NVML_NVLINK_ERROR_DL_REPLAY, &v) != NVML_SUCCESS) continue;  // link not present
    out->linksRead++;
    out->replay += v;
    if (gN.nvlinkError(h, link, NVML_NVLINK_ERROR_DL_RECOVERY, &v) == NVML_SUCCESS) out->recovery += v;
    if (gN.nvlinkError(h, link, NVML_NVLINK_ERROR_DL_CRC_FLIT, &v) == NVML_SUCCESS) out->crcFlit += v;
    if (gN.nvlinkError(h, link, NVML_NVLINK_ERROR_DL_CRC_DATA, &v) == NVML_SUCCESS) out->crcData += v;
  }
  return B200SMI_OK;
}

b200smi_status_t b200smi_pcie(int device, uint32_t* generation, uint32_t* width) {
  using namespace b200::smi;
  if (!generation || !width) return B200SMI_ERR_INVALID;
  nvmlDevice_t h;
  b200smi_status_t st = deviceHandle(device, &h);
  if (st != B200SMI_OK) return st;
  if (!gN.pcieGen || !gN.pcieWidth) return B200SMI_ERR_NOT_SUPPORTED;
  unsigned g = 0, w = 0;
  if (gN.pcieGen(h, &g) != NVML_SUCCESS || gN.pcieWidth(h, &w) != NVML_SUCCESS) return B200SMI_ERR_NVML;
  *generation = g;
  *width = w;
  return B200SMI_OK;
}

b200smi_status_t b200smi_modes(int device, b200smi_modes_t* out) {
  using namespace b200::smi;
  if (!out) return B200SMI_ERR_INVALID;
  nvmlDevice_t h;
  b200smi_status_t st = deviceHandle(device, &h);
  if (st != B200SMI_OK) return st;
  out->computeMode = out->persistence = out->mig = out->ecc = -1;
  nvmlComputeMode_t cm;
  if (gN.computeMode && gN.computeMode(h, &cm) == NVML_SUCCESS) out->computeMode = (int)cm;
  nvmlEnableState_t e, pending;
  if (gN.persistence && gN.persistence(h, &e) == NVML_SUCCESS) out->persistence = e == NVML_FEATURE_ENABLED;
  unsigned int cur = 0, pend = 0;
  if (gN.migMode && gN.migMode(h, &cur, &pend) == NVML_SUCCESS) out->mig = (int)cur;
  if (gN.eccMode && gN.eccMode(h, &e, &pending) == NVML_SUCCESS) out->ecc = e == NVML_FEATURE_ENABLED;
  return B200SMI_OK;
}

// ---- asynchronous events -------------------------------------------------------------------------------------------
// XID errors, ECC errors, power-state and clock changes as they happen, through one NVML event set over all devices:
// the counterpart of rsmi_event_notification_init / _mask_set / _get (rocm_smi_lib src/rocm_smi.cc:6116-6184), which the
// reference's health monitoring builds on. Read-only: nothing is acknowledged or cleared on the device.
namespace {
std::mutex gEvMu;
nvmlEventSet_t gEvSet = nullptr;
}  // namespace

b200smi_status_t b200smi_events_open(uint64_t mask) {
  using namespace b200::smi;
  if (!ready()) return B200SMI_ERR_NOT_LOADED;
  if (!gN.eventSetCreate || !gN.registerEvents || !gN.eventSetWait || !gN.eventSetFree) return B200SMI_ERR_NOT_SUPPORTED;
  std::lock_guard<std::mutex> lk(gEvMu);
  if (gEvSet) return B200SMI_OK;
  nvmlEventSet_t set = nullptr;
  if (gN.eventSetCreate(&set) != NVML_SUCCESS) return B200SMI_ERR_NVML;
  unsigned n = 0;
  gN.count(&n);
  int registered = 0;
  for (unsigned i = 0; i < n; i++) {
    nvmlDevice_t h;
    if (gN.handle(i, &h) != NVML_SUCCESS) continue;
    unsigned long long types = mask;
    unsigned long long supported = ~0ull;
    if (gN.supportedEvents && gN.supportedEvents(h, &supported) != NVML_SUCCESS) supported = 0;
    types = (mask ? mask : ~0ull) & supported;
    if (types && gN.registerEvents(h, types, set) == NVML_SUCCESS) registered++;
  }
  if (!registered) {
    gN.eventSetFree(set);
    return B200SMI_ERR_NOT_SUPPORTED;
  }
  gEvSet = set;
  return B200SMI_OK;
}

b200smi_status_t b200smi_events_wait(int timeoutMs, b200smi_event_t* out) {
  using namespace b200::smi;
  if (!out) return B200SMI_ERR_INVALID;
  nvmlEventSet_t set;
  {
    std::lock_guard<std::mutex> lk(gEvMu);
    set = gEvSet;
  }
  if (!set) return B200SMI_ERR_INVALID;
  nvmlEventData_t d;
  memset(&d, 0, sizeof(d));
  const nvmlReturn_t r = gN.eventSetWait(set, &d, timeoutMs < 0 ? 0 : (unsigned)timeoutMs);
  if (r == NVML_ERROR_TIMEOUT) return B200SMI_ERR_TIMEOUT;
  if (r != NVML_SUCCESS) return B200SMI_ERR_NVML;
  out->device = -1;
  unsigned n = 0;
  gN.count(&n);
  for (unsigned i = 0; i < n; i++) {
    nvmlDevice_t h;
    if (gN.handle(i, &h) == NVML_SUCCESS && h == d.device) out->device = (int)i;
  }
  out->type = d.eventType;
  out->data = d.eventData;
  timespec ts;
  clock_gettime(CLOCK_REALTIME, &ts);
  out->timestampNs = (uint64_t)ts.tv_sec * 1000000000ull + ts.tv_nsec;
  return B200SMI_OK;
}

b200smi_status_t b200smi_events_close(void) {
  using namespace b200::smi;
  std::lock_guard<std::mutex> lk(gEvMu);
  if (gEvSet && gN.eventSetFree) gN.eventSetFree(gEvSet);
  gEvSet = nullptr;
  return B200SMI_OK;
}

}  // extern "C"
