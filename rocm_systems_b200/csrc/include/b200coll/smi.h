/*
 * b200smi — device management, topology and telemetry C API (the role rocm-smi-lib and the RDC
 * library play in the reference: rocm-smi-lib/include/rocm_smi/rocm_smi.h, rdc/include/rdc/rdc.h).
 *
 * Readings come from NVML, loaded at run time (libnvidia-ml.so.1, or the library named by
 * B200SMI_NVML_LIBRARY — tests point this at a fake), and from the CUDA runtime for peer-to-peer
 * attributes. Nothing here changes a GPU setting unless B200SMI_ALLOW_SET=1 is in the environment
 * AND the caller passes allow = 1; the default is read-only.
 */
#ifndef B200COLL_SMI_H_
#define B200COLL_SMI_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  B200SMI_OK = 0,
  B200SMI_ERR_NOT_LOADED = 1,    /* NVML could not be loaded */
  B200SMI_ERR_INVALID = 2,
  B200SMI_ERR_NOT_SUPPORTED = 3,
  B200SMI_ERR_PERMISSION = 4,    /* a setter was called without being allowed */
  B200SMI_ERR_NVML = 5,
  B200SMI_ERR_TIMEOUT = 6        /* no event within the time given */
} b200smi_status_t;

typedef struct {
  char name[96];
  char uuid[96];
  char busId[32];
  uint32_t smClockMhz, smClockMaxMhz, memClockMhz, memClockMaxMhz;
  uint32_t powerMilliwatt, powerLimitMilliwatt;
  uint32_t temperatureC;
  uint64_t memTotalBytes, memUsedBytes;
  uint64_t eccCorrected, eccUncorrected;   /* volatile counters */
  uint64_t throttleReasons;                /* NVML clocks-event-reasons bit mask */
  uint32_t gpuUtilPct, memUtilPct;
  uint32_t nvlinkCount, nvlinkActive;      /* links the device has / links that are up */
  uint32_t multicastCapable;
} b200smi_device_info_t;

typedef enum { B200SMI_LINK_SELF = 0, B200SMI_LINK_NVLINK = 1, B200SMI_LINK_PCIE = 2, B200SMI_LINK_UNKNOWN = 3 } b200smi_link_type_t;

/* One directed edge of the device graph: the fields rocm-smi reports per GPU pair (type, hops,
 * weight, min/max bandwidth, P2P accessibility; rocm-smi-lib/src/rocm_smi.cc:4665-4910) plus the
 * atomics / coherency flags the runtime's link table carries
 * (rocr-runtime/runtime/hsa-runtime/core/runtime/amd_topology.cpp:188-258). */
typedef struct {
  int type;              /* b200smi_link_type_t */
  uint32_t hops;         /* 0 self, 1 through NVSwitch, 2+ over PCIe */
  uint32_t weight;       /* 0 self, 15 NVLink (one switch hop), 40 PCIe */
  uint32_t nvlinks;      /* bonded links between the pair (through the switch: all of the device's links) */
  uint64_t minBandwidthMBps, maxBandwidthMBps;
  int p2pAccessible, atomics32, atomics64, coherent;
  int perfRank;          /* cudaDevP2PAttrPerformanceRank, -1 unknown */
} b200smi_link_t;

typedef enum {
  B200SMI_FIELD_SM_CLOCK = 1, B200SMI_FIELD_MEM_CLOCK, B200SMI_FIELD_POWER, B200SMI_FIELD_TEMP, B200SMI_FIELD_MEM_USED,
  B200SMI_FIELD_GPU_UTIL, B200SMI_FIELD_MEM_UTIL, B200SMI_FIELD_ECC_CORRECTED, B200SMI_FIELD_ECC_UNCORRECTED,
  B200SMI_FIELD_THROTTLE_REASONS, B200SMI_FIELD_NVLINK_ACTIVE,
  /* Activity over the interval since the previous reading, from the driver's performance-monitoring samples (no
   * profiler attached, no replay): percentages of peak, and traffic in MiB/s. */
  B200SMI_FIELD_SM_ACTIVE, B200SMI_FIELD_SM_OCCUPANCY, B200SMI_FIELD_TENSOR_ACTIVE, B200SMI_FIELD_DRAM_ACTIVE,
  B200SMI_FIELD_FP64_ACTIVE, B200SMI_FIELD_FP32_ACTIVE, B200SMI_FIELD_FP16_ACTIVE,
  B200SMI_FIELD_PCIE_TX_MIBS, B200SMI_FIELD_PCIE_RX_MIBS, B200SMI_FIELD_NVLINK_TX_MIBS, B200SMI_FIELD_NVLINK_RX_MIBS,
  B200SMI_FIELD_COUNT_
} b200smi_field_t;

/* All activity readings of one device over one interval. A value the device does not report is negative. */
typedef struct {
  double intervalMs;
  double smActivePct, smOccupancyPct, tensorActivePct, dramActivePct, fp64ActivePct, fp32ActivePct, fp16ActivePct;
  double pcieTxMiBs, pcieRxMiBs, nvlinkTxMiBs, nvlinkRxMiBs;
} b200smi_activity_t;

typedef struct { uint64_t timestampNs; double value; } b200smi_sample_t;
typedef struct { double min, max, avg, last; uint64_t samples; } b200smi_stats_t;

/* Policy: fire `cb` when `field` of `device` goes above (dir > 0) or below (dir < 0) `threshold`. */
typedef void (*b200smi_policy_cb)(int device, int field, double value, double threshold, void* user);

b200smi_status_t b200smi_init(void);          /* ref-counted */
b200smi_status_t b200smi_shutdown(void);
const char* b200smi_status_string(b200smi_status_t s);
b200smi_status_t b200smi_device_count(int* count);
b200smi_status_t b200smi_device_info(int device, b200smi_device_info_t* info);
b200smi_status_t b200smi_read_field(int device, int field, double* value);
/* Activity between the previous call for this device and now. The first call (or one more than 5 s after the previous)
 * takes two samples 100 ms apart itself; calls less than 50 ms after the previous one return its result again.
 * B200SMI_ERR_NOT_SUPPORTED when the driver or the device has no performance-monitoring samples. */
b200smi_status_t b200smi_activity(int device, b200smi_activity_t* out);
b200smi_status_t b200smi_link(int from, int to, b200smi_link_t* link);
/* Driver version string, compute processes on a device, NVLink error counters summed over the
 * device's links, and the PCIe link it trains at (rocm-smi: --showdriverversion, --showpids,
 * rsmi_dev_xgmi_error_status, --showbus). */
typedef struct { uint32_t pid; uint64_t usedMemoryBytes; char name[64]; } b200smi_process_t;
typedef struct { uint64_t replay, recovery, crcFlit, crcData; uint32_t linksRead; } b200smi_nvlink_errors_t;
b200smi_status_t b200smi_driver_version(char* buf, int len);
b200smi_status_t b200smi_processes(int device, b200smi_process_t* out, int max, int* n);
b200smi_status_t b200smi_nvlink_errors(int device, b200smi_nvlink_errors_t* out);
b200smi_status_t b200smi_pcie(int device, uint32_t* generation, uint32_t* width);
/* Modes of a device, read only (this library never changes them): compute mode (0 default, 1 exclusive thread, 2 prohibited,
 * 3 exclusive process), persistence, MIG and ECC enabled flags; -1 where the driver does not report one. */
typedef struct { int computeMode, persistence, mig, ecc; } b200smi_modes_t;
b200smi_status_t b200smi_modes(int device, b200smi_modes_t* out);

/* Identity and lifetime readings (rocm-smi: --showserial, --showvbios, --showperflevel, --showmaxpower, --showenergycounter,
 * --showretiredpages): serial and part numbers, firmware versions, performance state (0 = fastest), the range the power limit
 * may be set in, energy drawn since the driver was loaded, and rows of device memory remapped after errors. A string the
 * driver does not report is empty, a number is -1. */
typedef struct {
  char serial[32], partNumber[64], vbios[32], inforomImage[32];
  int performanceState;
  int64_t powerLimitMinMilliwatt, powerLimitMaxMilliwatt;
  int64_t energyMillijoule;
  int remappedCorrectable, remappedUncorrectable, remapPending, remapFailed;
} b200smi_identity_t;
b200smi_status_t b200smi_identity(int device, b200smi_identity_t* out);

/* CPUs and NUMA node a device is attached to (rocm-smi: --showtoponuma, rsmi_topo_get_numa_node_number /
 * rsmi_topo_numa_affinity_get): `mask` receives one bit per logical CPU, 64 per word, as many words as given; numaNode is -1
 * when the driver does not say. A process that drives this GPU runs best on these CPUs. */
b200smi_status_t b200smi_cpu_affinity(int device, uint64_t* mask, int words, int* numaNode);

/* Asynchronous events of all devices (read only). Types are NVML's bits. */
#define B200SMI_EVENT_ECC_SINGLE 0x1ull
#define B200SMI_EVENT_ECC_DOUBLE 0x2ull
#define B200SMI_EVENT_PSTATE 0x4ull
#define B200SMI_EVENT_XID 0x8ull          /* data = the XID number */
#define B200SMI_EVENT_CLOCK 0x10ull
#define B200SMI_EVENT_POWER_SOURCE 0x80ull
typedef struct { int device; uint64_t type; uint64_t data; uint64_t timestampNs; } b200smi_event_t;
b200smi_status_t b200smi_events_open(uint64_t mask);                       /* 0: every type a device supports */
b200smi_status_t b200smi_events_wait(int timeoutMs, b200smi_event_t* out);  /* B200SMI_ERR_TIMEOUT when nothing happened */
b200smi_status_t b200smi_events_close(void);
/* Watches: a sampler thread reads the watched fields every periodMs into a per-(device, field)
 * ring of `keep` samples (the watch table and cache of rdc_libs/rdc/src/RdcWatchTableImpl.cc). */
b200smi_status_t b200smi_watch_start(const int* devices, int ndev, const int* fields, int nfields, int periodMs, int keep);
b200smi_status_t b200smi_watch_stop(void);
b200smi_status_t b200smi_watch_latest(int device, int field, b200smi_sample_t* out);
b200smi_status_t b200smi_watch_history(int device, int field, b200smi_sample_t* out, int max, int* n);
/* Job statistics: min / max / average of every watched field between start and stop. */
b200smi_status_t b200smi_job_start(const char* jobId);
b200smi_status_t b200smi_job_stop(const char* jobId);
b200smi_status_t b200smi_job_stats(const char* jobId, int device, int field, b200smi_stats_t* out);
b200smi_status_t b200smi_policy_set(int device, int field, double threshold, int dir, b200smi_policy_cb cb, void* user);
b200smi_status_t b200smi_policy_clear(void);
/* Health: 0 pass, 1 warn, 2 fail, with a short reason (ECC, throttling, NVLink down, temperature). */
b200smi_status_t b200smi_health(int device, int* level, char* reason, int reasonLen);
/* Setter (off unless allowed twice, see the top of this header). */
b200smi_status_t b200smi_set_power_limit(int device, uint32_t milliwatt, int allow);
/* Locks the SM clock into [minMhz, maxMhz], or (reset) hands it back to the driver. The same double gate as the power limit;
 * a lock outlasts the process, so whoever sets one resets it. */
b200smi_status_t b200smi_set_locked_clocks(int device, uint32_t minMhz, uint32_t maxMhz, int allow);
b200smi_status_t b200smi_reset_locked_clocks(int device, int allow);

#ifdef __cplusplus
}
#endif

#endif /* B200COLL_SMI_H_ */
