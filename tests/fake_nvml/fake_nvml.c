/* A stand-in for libnvidia-ml used by the CPU tests of b200smi: a fixed fleet of FAKE_NVML_GPUS
 * (default 8) "B200" devices with 18 NVLinks each. Environment knobs change what it reports:
 *   FAKE_NVML_LINK_DOWN=<gpu>      one link of that GPU is reported down
 *   FAKE_NVML_ECC=<gpu>            that GPU reports 3 uncorrected ECC errors
 *   FAKE_NVML_TEMP=<celsius>       temperature of every GPU
 *   FAKE_NVML_RAMP=1               power rises by 10 W on every read (for watch / policy tests)
 *   FAKE_NVML_EVENTS=<gpu>:<type>:<data>[,...]   events the event set hands out, one per wait, then time-outs
 *   FAKE_NVML_GPM=0                the performance-monitoring samples are reported as unsupported
 *   FAKE_NVML_TENSOR=<percent>     tensor activity every GPU reports (default 62.5); NVLink traffic is 1000 MiB/s per
 *                                  sample taken between the two samples of a request, so it shows which pair was used
 * The last power limit a setter wrote is kept in memory and returned by the getter. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

typedef struct fake_dev { int idx; } *nvmlDevice_t;
typedef int nvmlReturn_t;
#define NVML_SUCCESS 0
#define NVML_ERROR_INVALID_ARGUMENT 2
typedef struct { char busIdLegacy[16]; unsigned int domain, bus, device, pciDeviceId, pciSubSystemId; char busId[32]; } nvmlPciInfo_t;
typedef struct { unsigned long long total, free, used; } nvmlMemory_t;
typedef struct { unsigned int gpu, memory; } nvmlUtilization_t;

static struct fake_dev devs[16];
static unsigned int power_limit[16];
static unsigned int reads = 0;

static int ngpus(void) { const char* e = getenv("FAKE_NVML_GPUS"); int n = e ? atoi(e) : 8; return n < 1 ? 1 : (n > 16 ? 16 : n); }
static int envint(const char* k, int d) { const char* e = getenv(k); return e ? atoi(e) : d; }

nvmlReturn_t nvmlInit_v2(void) { for (int i = 0; i < 16; i++) { devs[i].idx = i; if (!power_limit[i]) power_limit[i] = 1000000; } return NVML_SUCCESS; }
nvmlReturn_t nvmlShutdown(void) { return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetCount_v2(unsigned int* n) { *n = (unsigned)ngpus(); return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetHandleByIndex_v2(unsigned int i, nvmlDevice_t* d) { if ((int)i >= ngpus()) return NVML_ERROR_INVALID_ARGUMENT; *d = &devs[i]; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetName(nvmlDevice_t d, char* s, unsigned int n) { (void)d; snprintf(s, n, "NVIDIA B200 (fake)"); return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetUUID(nvmlDevice_t d, char* s, unsigned int n) { snprintf(s, n, "GPU-fake-%04d", d->idx); return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetPciInfo_v3(nvmlDevice_t d, nvmlPciInfo_t* p) { memset(p, 0, sizeof(*p)); snprintf(p->busId, sizeof(p->busId), "00000000:%02X:00.0", 0x10 + d->idx); return NVML_SUCCESS; }
static unsigned int locked_max[16];
nvmlReturn_t nvmlDeviceGetClockInfo(nvmlDevice_t d, int t, unsigned int* c) { *c = t == 1 /*SM*/ ? (locked_max[d->idx] ? locked_max[d->idx] : 1500) : 3996; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetMaxClockInfo(nvmlDevice_t d, int t, unsigned int* c) { (void)d; *c = t == 1 ? 1965 : 3996; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetPowerUsage(nvmlDevice_t d, unsigned int* mw) { (void)d; reads++; *mw = 200000 + (envint("FAKE_NVML_RAMP", 0) ? reads * 10000 : 0); return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetEnforcedPowerLimit(nvmlDevice_t d, unsigned int* mw) { *mw = power_limit[d->idx]; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceSetPowerManagementLimit(nvmlDevice_t d, unsigned int mw) { power_limit[d->idx] = mw; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetTemperature(nvmlDevice_t d, int s, unsigned int* t) { (void)d; (void)s; *t = (unsigned)envint("FAKE_NVML_TEMP", 45); return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetMemoryInfo(nvmlDevice_t d, nvmlMemory_t* m) { (void)d; m->total = 183359ull << 20; m->used = 1024ull << 20; m->free = m->total - m->used; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetTotalEccErrors(nvmlDevice_t d, int type, int counter, unsigned long long* c) { (void)counter; *c = (type == 1 /*uncorrected*/ && envint("FAKE_NVML_ECC", -1) == d->idx) ? 3 : 0; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetCurrentClocksEventReasons(nvmlDevice_t d, unsigned long long* r) { (void)d; *r = 0x4; /* sw power cap */ return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetUtilizationRates(nvmlDevice_t d, nvmlUtilization_t* u) { (void)d; u->gpu = 97; u->memory = 40; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetNvLinkState(nvmlDevice_t d, unsigned int link, int* active) { if (link >= 18) return NVML_ERROR_INVALID_ARGUMENT; *active = !(envint("FAKE_NVML_LINK_DOWN", -1) == d->idx && link == 5); return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetNvLinkRemotePciInfo_v2(nvmlDevice_t d, unsigned int link, nvmlPciInfo_t* p) { (void)d; (void)link; memset(p, 0, sizeof(*p)); snprintf(p->busId, sizeof(p->busId), "00000000:F0:00.0"); return NVML_SUCCESS; }

/* driver version, processes, NVLink error counters, PCIe link */
typedef struct { unsigned int pid; unsigned long long usedGpuMemory; unsigned int gpuInstanceId, computeInstanceId; } nvmlProcessInfo_t;
nvmlReturn_t nvmlSystemGetDriverVersion(char* s, unsigned int n) { snprintf(s, n, "580.159.fake"); return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetComputeRunningProcesses_v3(nvmlDevice_t d, unsigned int* count, nvmlProcessInfo_t* infos) {
  /* GPU 0 runs two processes (this one and pid 1), the others none */
  unsigned int have = d->idx == 0 ? 2 : 0;
  if (*count < have) { *count = have; return 7; /* NVML_ERROR_INSUFFICIENT_SIZE */ }
  *count = have;
  if (have) {
    memset(infos, 0, have * sizeof(*infos));
    infos[0].pid = (unsigned)getpid(); infos[0].usedGpuMemory = 3ull << 30;
    infos[1].pid = 1; infos[1].usedGpuMemory = 1ull << 30;
  }
  return NVML_SUCCESS;
}
nvmlReturn_t nvmlDeviceGetNvLinkErrorCounter(nvmlDevice_t d, unsigned int link, int counter, unsigned long long* v) {
  if (link >= 18) return NVML_ERROR_INVALID_ARGUMENT;
  /* FAKE_NVML_LINK_ERRORS=<gpu>: that GPU shows 5 replays on link 3 */
  *v = (envint("FAKE_NVML_LINK_ERRORS", -1) == d->idx && link == 3 && counter == 0) ? 5 : 0;
  return NVML_SUCCESS;
}
nvmlReturn_t nvmlDeviceGetCurrPcieLinkGeneration(nvmlDevice_t d, unsigned int* g) { (void)d; *g = 5; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetCurrPcieLinkWidth(nvmlDevice_t d, unsigned int* w) { (void)d; *w = 16; return NVML_SUCCESS; }

/* modes (read only) */
nvmlReturn_t nvmlDeviceGetComputeMode(nvmlDevice_t d, int* m) { (void)d; *m = 0; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetPersistenceMode(nvmlDevice_t d, int* e) { (void)d; *e = 1; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetMigMode(nvmlDevice_t d, unsigned int* cur, unsigned int* pend) { (void)d; *cur = 0; *pend = 0; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetEccMode(nvmlDevice_t d, int* cur, int* pend) { (void)d; *cur = 1; *pend = 1; return NVML_SUCCESS; }

/* events: a set hands out the FAKE_NVML_EVENTS list in order, one per wait, for devices registered with a matching type */
typedef struct fake_set { unsigned long long types[16]; int next; } *nvmlEventSet_t;
typedef struct { nvmlDevice_t device; unsigned long long eventType, eventData; unsigned int gpuInstanceId, computeInstanceId; } nvmlEventData_t;
static struct fake_set the_set;
nvmlReturn_t nvmlEventSetCreate(nvmlEventSet_t* s) { memset(&the_set, 0, sizeof(the_set)); *s = &the_set; return NVML_SUCCESS; }
nvmlReturn_t nvmlEventSetFree(nvmlEventSet_t s) { (void)s; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetSupportedEventTypes(nvmlDevice_t d, unsigned long long* t) { (void)d; *t = 0x1f; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceRegisterEvents(nvmlDevice_t d, unsigned long long types, nvmlEventSet_t s) { s->types[d->idx] |= types; return NVML_SUCCESS; }
nvmlReturn_t nvmlEventSetWait_v2(nvmlEventSet_t s, nvmlEventData_t* out, unsigned int timeoutms) {
  const char* e = getenv("FAKE_NVML_EVENTS");
  int k = 0;
  while (e && *e) {
    int gpu = 0;
    unsigned long long type = 0, data = 0;
    if (sscanf(e, "%d:%llu:%llu", &gpu, &type, &data) != 3) break;
    if (k++ >= s->next) {
      s->next = k;
      if (gpu >= 0 && gpu < 16 && (s->types[gpu] & type)) {
        out->device = &devs[gpu]; out->eventType = type; out->eventData = data; out->gpuInstanceId = out->computeInstanceId = 0xffffffffu;
        return NVML_SUCCESS;
      }
    }
    e = strchr(e, ',');
    if (e) e++;
  }
  usleep((timeoutms > 50 ? 50 : timeoutms) * 1000);
  return 10; /* NVML_ERROR_TIMEOUT */
}

/* ---- CPU affinity: GPU i sits on CPUs [4 i, 4 i + 3] (FAKE_NVML_CPUS_PER_GPU changes the 4), four GPUs per NUMA node ---- */
nvmlReturn_t nvmlDeviceGetCpuAffinity(nvmlDevice_t d, unsigned int words, unsigned long* set) {
  int per = envint("FAKE_NVML_CPUS_PER_GPU", 4);
  memset(set, 0, sizeof(unsigned long) * words);
  for (int c = d->idx * per; c < (d->idx + 1) * per; c++)
    if ((unsigned)(c / 64) < words) set[c / 64] |= 1ul << (c % 64);
  return NVML_SUCCESS;
}
nvmlReturn_t nvmlDeviceGetNumaNodeId(nvmlDevice_t d, unsigned int* node) { *node = (unsigned)(d->idx / 4); return NVML_SUCCESS; }

/* ---- identity, lifetime counters, clock locks (kept in memory, shown by the clock getter) ---- */
static unsigned int locked_min[16];
nvmlReturn_t nvmlDeviceGetSerial(nvmlDevice_t d, char* s, unsigned int n) { snprintf(s, n, "165012345%04d", d->idx); return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetBoardPartNumber(nvmlDevice_t d, char* s, unsigned int n) { (void)d; snprintf(s, n, "699-2G525-0200-000"); return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetVbiosVersion(nvmlDevice_t d, char* s, unsigned int n) { (void)d; snprintf(s, n, "97.00.88.00.0F"); return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetInforomImageVersion(nvmlDevice_t d, char* s, unsigned int n) { (void)d; (void)s; (void)n; return 3; /* not supported */ }
nvmlReturn_t nvmlDeviceGetPerformanceState(nvmlDevice_t d, int* p) { (void)d; *p = 0; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetPowerManagementLimitConstraints(nvmlDevice_t d, unsigned int* lo, unsigned int* hi) { (void)d; *lo = 200000; *hi = 1000000; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetTotalEnergyConsumption(nvmlDevice_t d, unsigned long long* mj) { *mj = 123456789ull + (unsigned long long)d->idx; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceGetRemappedRows(nvmlDevice_t d, unsigned int* c, unsigned int* u, unsigned int* pend, unsigned int* fail) {
  *c = envint("FAKE_NVML_ECC", -1) == d->idx ? 2 : 0; *u = 0; *pend = 0; *fail = 0; return NVML_SUCCESS;
}
nvmlReturn_t nvmlDeviceSetGpuLockedClocks(nvmlDevice_t d, unsigned int lo, unsigned int hi) { locked_min[d->idx] = lo; locked_max[d->idx] = hi; return NVML_SUCCESS; }
nvmlReturn_t nvmlDeviceResetGpuLockedClocks(nvmlDevice_t d) { locked_min[d->idx] = locked_max[d->idx] = 0; return NVML_SUCCESS; }

/* ---- performance-monitoring samples: a sample remembers its sequence number; a metrics request reports fixed
 * percentages, the number of samples between its two samples as NVLink traffic, and "not available" for FP64. ---- */
typedef struct fake_sample { int seq; } *nvmlGpmSample_t;
typedef struct { unsigned int version; unsigned int isSupportedDevice; } nvmlGpmSupport_t;
typedef struct { unsigned int metricId; nvmlReturn_t nvmlReturn; double value; struct { char* shortName; char* longName; char* unit; } metricInfo; } nvmlGpmMetric_t;
#define FAKE_GPM_METRIC_MAX 210
typedef struct { unsigned int version; unsigned int numMetrics; nvmlGpmSample_t sample1, sample2; nvmlGpmMetric_t metrics[FAKE_GPM_METRIC_MAX]; } nvmlGpmMetricsGet_t;
static int sample_seq = 0;
nvmlReturn_t nvmlGpmQueryDeviceSupport(nvmlDevice_t d, nvmlGpmSupport_t* s) { (void)d; s->isSupportedDevice = envint("FAKE_NVML_GPM", 1) ? 1 : 0; return NVML_SUCCESS; }
nvmlReturn_t nvmlGpmSampleAlloc(nvmlGpmSample_t* s) { *s = calloc(1, sizeof(struct fake_sample)); return *s ? NVML_SUCCESS : 20; }
nvmlReturn_t nvmlGpmSampleFree(nvmlGpmSample_t s) { free(s); return NVML_SUCCESS; }
nvmlReturn_t nvmlGpmSampleGet(nvmlDevice_t d, nvmlGpmSample_t s) { (void)d; s->seq = ++sample_seq; return NVML_SUCCESS; }
nvmlReturn_t nvmlGpmMetricsGet(nvmlGpmMetricsGet_t* r) {
  if (r->version != 1 || !r->sample1 || !r->sample2 || r->sample2->seq <= r->sample1->seq) return NVML_ERROR_INVALID_ARGUMENT;
  const char* t = getenv("FAKE_NVML_TENSOR");
  for (unsigned i = 0; i < r->numMetrics; i++) {
    nvmlGpmMetric_t* m = &r->metrics[i];
    m->nvmlReturn = NVML_SUCCESS;
    switch (m->metricId) {
      case 2: m->value = 91.0; break;                       /* SM busy */
      case 3: m->value = 48.5; break;                       /* occupancy */
      case 5: m->value = t ? atof(t) : 62.5; break;         /* any tensor */
      case 10: m->value = 33.0; break;                      /* DRAM */
      case 11: m->nvmlReturn = 3; m->value = 0; break;      /* FP64: not available */
      case 12: m->value = 7.0; break;
      case 13: m->value = 1.0; break;
      case 20: m->value = 120.0; break;
      case 21: m->value = 80.0; break;
      case 60: m->value = 900.0 * (r->sample2->seq - r->sample1->seq); break;   /* NVLink RX */
      case 61: m->value = 1000.0 * (r->sample2->seq - r->sample1->seq); break;  /* NVLink TX */
      default: m->nvmlReturn = NVML_ERROR_INVALID_ARGUMENT; break;
    }
  }
  return NVML_SUCCESS;
}
