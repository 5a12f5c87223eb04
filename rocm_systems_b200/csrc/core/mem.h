// Symmetric memory: allocations that every rank of a communicator maps, plus the NVSwitch
// multicast alias used by the multimem (NVLS) kernels.
//
// The reference runtime builds the same thing from IPC handles and its virtual-memory API
// (rocr-runtime/runtime/hsa-runtime/core/runtime/runtime.cpp:1199-1545 IPC create/attach,
// :3147-3760 reserve/create/map/set-access/export/import). Here: cuMemCreate with a POSIX file
// descriptor handle, descriptors passed between ranks with SCM_RIGHTS, every rank's allocation
// mapped into one address reservation, and one multicast object bound to all of them. A legacy
// mode (cudaIpc handles, no multicast) exists for boxes where descriptor export is refused.
#pragma once

#include <cuda.h>

#include <map>
#include <mutex>

#include "bootstrap.h"
#include "common.h"

namespace b200 {

struct SymSeg {
  size_t size = 0;                  // mapped bytes per rank
  int nranks = 0, rank = -1;
  char* peer[kMaxRanks] = {};       // this rank's mapping of every rank's memory; peer[rank] is local
  char* mc = nullptr;               // multicast alias, or null
  bool legacy = false;              // cudaIpc mode
  bool ownsLocal = true;            // false when the local memory came from ncclMemAlloc
  // VMM bookkeeping
  CUmemGenericAllocationHandle handle[kMaxRanks] = {};
  CUmemGenericAllocationHandle mcHandle = 0;
  CUdeviceptr vaBase = 0;           // reservation holding the peer mappings
  size_t vaStride = 0;
  CUdeviceptr mcVa = 0;
  bool mcBound = false;
  void* legacyBase[kMaxRanks] = {}; // what cudaIpcOpenMemHandle returned (legacy mode)
};

struct MemCaps {
  bool vmm = false;         // cuMem* with POSIX fd handles usable
  bool multicast = false;   // device reports multicast support
  size_t allocGran = 2u << 20;
  size_t mcGran = 2u << 20;
};
ncclResult_t queryMemCaps(int cudaDev, MemCaps* caps);

// Collective over `boot`: allocate `bytes` (rounded up) on every rank and map all of them.
// `wantMc` asks for the multicast alias; it is dropped (on every rank alike) if any rank fails
// to set it up. `tag` must be the same on every rank and unique per call on this bootstrap.
ncclResult_t symAlloc(Bootstrap& boot, int cudaDev, size_t bytes, bool wantMc, uint32_t tag, SymSeg* seg);
// Collective: the same for memory that already exists locally (from ncclMemAlloc).
ncclResult_t symAdopt(Bootstrap& boot, int cudaDev, void* localBase, size_t bytes, bool wantMc, uint32_t tag, SymSeg* seg);
ncclResult_t symFree(SymSeg* seg, int cudaDev);

// ncclMemAlloc / ncclMemFree: exportable local allocations, tracked process-wide.
struct LocalAlloc {
  void* ptr;
  size_t size;      // mapped size (granularity multiple)
  int dev;
  CUmemGenericAllocationHandle handle;
  bool vmm;
};
ncclResult_t localAllocExportable(void** ptr, size_t size);
ncclResult_t localFreeExportable(void* ptr);
bool localAllocLookup(const void* ptr, LocalAlloc* out);  // finds the allocation containing ptr

}  // namespace b200
