// Shared between the two halves of b200smi (topo.cc, health.cc).
#pragma once

#include <nvml.h>

#include "b200coll/smi.h"

namespace b200 {
namespace smi {

struct NvmlFns {
  nvmlReturn_t (*init)(void) = nullptr;
  nvmlReturn_t (*shutdown)(void) = nullptr;
  nvmlReturn_t (*count)(unsigned int*) = nullptr;
  nvmlReturn_t (*handle)(unsigned int, nvmlDevice_t*) = nullptr;
  nvmlReturn_t (*name)(nvmlDevice_t, char*, unsigned int) = nullptr;
  nvmlReturn_t (*uuid)(nvmlDevice_t, char*, unsigned int) = nullptr;
  nvmlReturn_t (*pci)(nvmlDevice_t, nvmlPciInfo_t*) = nullptr;
  nvmlReturn_t (*clock)(nvmlDevice_t, nvmlClockType_t, unsigned int*) = nullptr;
  nvmlReturn_t (*maxClock)(nvmlDevice_t, nvmlClockType_t, unsigned int*) = nullptr;
  nvmlReturn_t (*power)(nvmlDevice_t, unsigned int*) = nullptr;
  nvmlReturn_t (*powerLimit)(nvmlDevice_t, unsigned int*) = nullptr;
  nvmlReturn_t (*temp)(nvmlDevice_t, nvmlTemperatureSensors_t, unsigned int*) = nullptr;
  nvmlReturn_t (*mem)(nvmlDevice_t, nvmlMemory_t*) = nullptr;
  nvmlReturn_t (*ecc)(nvmlDevice_t, nvmlMemoryErrorType_t, nvmlEccCounterType_t, unsigned long long*) = nullptr;
  nvmlReturn_t (*reasons)(nvmlDevice_t, unsigned long long*) = nullptr;
  nvmlReturn_t (*util)(nvmlDevice_t, nvmlUtilization_t*) = nullptr;
  nvmlReturn_t (*nvlinkState)(nvmlDevice_t, unsigned int, nvmlEnableState_t*) = nullptr;
  nvmlReturn_t (*nvlinkRemote)(nvmlDevice_t, unsigned int, nvmlPciInfo_t*) = nullptr;
  nvmlReturn_t (*setPowerLimit)(nvmlDevice_t, unsigned int) = nullptr;
  nvmlReturn_t (*driverVersion)(char*, unsigned int) = nullptr;
  nvmlReturn_t (*processes)(nvmlDevice_t, unsigned int*, nvmlProcessInfo_t*) = nullptr;
  nvmlReturn_t (*nvlinkError)(nvmlDevice_t, unsigned int, nvmlNvLinkErrorCounter_t, unsigned long long*) = nullptr;
  nvmlReturn_t (*pcieGen)(nvmlDevice_t, unsigned int*) = nullptr;
  nvmlReturn_t (*pcieWidth)(nvmlDevice_t, unsigned int*) = nullptr;
  nvmlReturn_t (*computeMode)(nvmlDevice_t, nvmlComputeMode_t*) = nullptr;
  nvmlReturn_t (*persistence)(nvmlDevice_t, nvmlEnableState_t*) = nullptr;
  nvmlReturn_t (*migMode)(nvmlDevice_t, unsigned int*, unsigned int*) = nullptr;
  nvmlReturn_t (*eccMode)(nvmlDevice_t, nvmlEnableState_t*, nvmlEnableState_t*) = nullptr;
  nvmlReturn_t (*eventSetCreate)(nvmlEventSet_t*) = nullptr;
  nvmlReturn_t (*eventSetFree)(nvmlEventSet_t) = nullptr;
  nvmlReturn_t (*supportedEvents)(nvmlDevice_t, unsigned long long*) = nullptr;
  nvmlReturn_t (*registerEvents)(nvmlDevice_t, unsigned long long, nvmlEventSet_t) = nullptr;
  nvmlReturn_t (*eventSetWait)(nvmlEventSet_t, nvmlEventData_t*, unsigned int) = nullptr;
  nvmlReturn_t (*cpuAffinity)(nvmlDevice_t, unsigned int, unsigned long*) = nullptr;
  nvmlReturn_t (*numaNode)(nvmlDevice_t, unsigned int*) = nullptr;
  nvmlReturn_t (*serial)(nvmlDevice_t, char*, unsigned int) = nullptr;
  nvmlReturn_t (*partNumber)(nvmlDevice_t, char*, unsigned int) = nullptr;
  nvmlReturn_t (*vbios)(nvmlDevice_t, char*, unsigned int) = nullptr;
  nvmlReturn_t (*inforomImage)(nvmlDevice_t, char*, unsigned int) = nullptr;
  nvmlReturn_t (*pstate)(nvmlDevice_t, nvmlPstates_t*) = nullptr;
  nvmlReturn_t (*powerConstraints)(nvmlDevice_t, unsigned int*, unsigned int*) = nullptr;
  nvmlReturn_t (*energy)(nvmlDevice_t, unsigned long long*) = nullptr;
  nvmlReturn_t (*remappedRows)(nvmlDevice_t, unsigned int*, unsigned int*, unsigned int*, unsigned int*) = nullptr;
  nvmlReturn_t (*setLockedClocks)(nvmlDevice_t, unsigned int, unsigned int) = nullptr;
  nvmlReturn_t (*resetLockedClocks)(nvmlDevice_t) = nullptr;
  nvmlReturn_t (*gpmSupport)(nvmlDevice_t, nvmlGpmSupport_t*) = nullptr;
  nvmlReturn_t (*gpmSampleAlloc)(nvmlGpmSample_t*) = nullptr;
  nvmlReturn_t (*gpmSampleFree)(nvmlGpmSample_t) = nullptr;
  nvmlReturn_t (*gpmSampleGet)(nvmlDevice_t, nvmlGpmSample_t) = nullptr;
  nvmlReturn_t (*gpmMetricsGet)(nvmlGpmMetricsGet_t*) = nullptr;
};
extern NvmlFns gN;
bool ready();
b200smi_status_t deviceHandle(int device, nvmlDevice_t* h);
void activityReset();     // topo.cc: frees the activity samples (called at the last shutdown)
void watchStopLocked();  // health.cc: stops the sampler thread (called at the last shutdown)

}  // namespace smi
}  // namespace b200
