#include "mem.h"

#include <string.h>
#include <unistd.h>

#include <vector>

#include "cudrv.h"

namespace b200 {

static size_t roundUp(size_t v, size_t g) { return (v + g - 1) / g * g; }

ncclResult_t queryMemCaps(int cudaDev, MemCaps* caps) {
  *caps = MemCaps();
  const CuDrv& d = CuDrv::get();
  if (!d.ok) return ncclSuccess;
  CUdevice cuDev;
  BCU(d.cuDeviceGet(&cuDev, cudaDev));
  int vmm = 0, fd = 0, mc = 0;
  d.cuDeviceGetAttribute(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, cuDev);
  d.cuDeviceGetAttribute(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cuDev);
  d.cuDeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cuDev);
  caps->vmm = vmm && fd;
  caps->multicast = caps->vmm && mc;
  if (caps->vmm) {
    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = cudaDev;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t g = 0;
    if (d.cuMemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && g) caps->allocGran = g;
  }
  if (caps->multicast) {
    CUmulticastObjectProp mp{};
    mp.numDevices = 2;
    mp.size = caps->allocGran;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t g = 0;
    if (d.cuMulticastGetGranularity(&g, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) == CUDA_SUCCESS && g) caps->mcGran = g;
    else caps->multicast = false;
  }
  return ncclSuccess;
}

// True on every rank iff `mine` is true on every rank.
static ncclResult_t allAgree(Bootstrap& boot, bool mine, bool* all) {
  std::vector<int> v(boot.nranks());
  int m = mine ? 1 : 0;
  BCHECK(boot.allGather(&m, v.data(), sizeof(int)));
  *all = true;
  for (int x : v) if (!x) *all = false;
  return ncclSuccess;
}

static void dropMc(SymSeg* seg) {
  const CuDrv& d = CuDrv::get();
  if (seg->mcVa) {
    d.cuMemUnmap(seg->mcVa, seg->size);
    d.cuMemAddressFree(seg->mcVa, seg->size);
    seg->mcVa = 0;
  }
  if (seg->mcHandle) {
    d.cuMemRelease(seg->mcHandle);
    seg->mcHandle = 0;
  }
  seg->mc = nullptr;
  seg->mcBound = false;
}

// Multicast set-up. Never returns an error for a box that merely cannot do it: every step's
// outcome is agreed between the ranks and all of them fall back together.
static ncclResult_t setupMulticast(Bootstrap& boot, int cudaDev, uint32_t tag, SymSeg* seg) {
  const CuDrv& d = CuDrv::get();
  const int n = boot.nranks(), rank = boot.rank();
  CUdevice cuDev;
  bool ok = d.cuDeviceGet(&cuDev, cudaDev) == CUDA_SUCCESS;
  bool all = false;
  int fd = -1;
  if (ok && rank == 0) {
    CUmulticastObjectProp mp{};
    mp.numDevices = (unsigned)n;
    mp.size = seg->size;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUresult r = d.cuMulticastCreate(&seg->mcHandle, &mp);
    if (r == CUDA_SUCCESS) r = d.cuMemExportToShareableHandle(&fd, seg->mcHandle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) {
      BINFO(SUB_MEM, "multicast object not available: %s", cuErrStr(r));
      ok = false;
    }
  }
  BCHECK(allAgree(boot, ok, &all));
  if (!all) { if (fd >= 0) ::close(fd); dropMc(seg); return ncclSuccess; }
  if (rank == 0) {
    for (int p = 1; p < n; p++) BCHECK(boot.sendFd(p, fd, tag));
    ::close(fd);
  } else {
    BCHECK(boot.recvFd(0, tag, &fd));
    CUresult r = d.cuMemImportFromShareableHandle(&seg->mcHandle, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    ::close(fd);
    if (r != CUDA_SUCCESS) { BINFO(SUB_MEM, "multicast import failed: %s", cuErrStr(r)); ok = false; }
  }
  if (ok) {
    CUresult r = d.cuMulticastAddDevice(seg->mcHandle, cuDev);
    if (r != CUDA_SUCCESS) { BINFO(SUB_MEM, "cuMulticastAddDevice failed: %s", cuErrStr(r)); ok = false; }
  }
  BCHECK(allAgree(boot, ok, &all));  // every device must be added before anyone binds
  if (!all) { dropMc(seg); return ncclSuccess; }
  {
    CUresult r = d.cuMulticastBindMem(seg->mcHandle, 0, seg->handle[rank], 0, seg->size, 0);
    if (r != CUDA_SUCCESS) { BINFO(SUB_MEM, "cuMulticastBindMem failed: %s", cuErrStr(r)); ok = false; }
    else seg->mcBound = true;
  }
  if (ok) {
    CUresult r = d.cuMemAddressReserve(&seg->mcVa, seg->size, 0, 0, 0);
    if (r == CUDA_SUCCESS) {
      r = d.cuMemMap(seg->mcVa, seg->size, 0, seg->mcHandle, 0);
      if (r == CUDA_SUCCESS) {
        CUmemAccessDesc ad{};
        ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        ad.location.id = cudaDev;
        ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        r = d.cuMemSetAccess(seg->mcVa, seg->size, &ad, 1);
      }
    }
    if (r != CUDA_SUCCESS) { BINFO(SUB_MEM, "multicast mapping failed: %s", cuErrStr(r)); ok = false; }
  }
  BCHECK(allAgree(boot, ok, &all));
  if (!all) { dropMc(seg); return ncclSuccess; }
  seg->mc = (char*)seg->mcVa;
  BINFO(SUB_MEM, "rank %d: multicast alias %p over %zu bytes", rank, (void*)seg->mc, seg->size);
  return ncclSuccess;
}

static ncclResult_t mapExchangeVmm(Bootstrap& boot, int cudaDev, CUmemGenericAllocationHandle mine, void* localPtr,
                                   size_t size, bool wantMc, uint32_t tag, SymSeg* seg) {
  const CuDrv& d = CuDrv::get();
  const int n = boot.nranks(), rank = boot.rank();
  seg->size = size;
  seg->nranks = n;
  seg->rank = rank;
  seg->handle[rank] = mine;
  int fd = -1;
  BCU(d.cuMemExportToShareableHandle(&fd, mine, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  for (int i = 1; i < n; i++) {
    int p = (rank + i) % n;
    ncclResult_t r = boot.sendFd(p, fd, tag);
    if (r != ncclSuccess) { ::close(fd); return r; }
  }
  ::close(fd);
  seg->vaStride = size;
  BCU(d.cuMemAddressReserve(&seg->vaBase, size * n, 0, 0, 0));
  for (int i = 0; i < n; i++) {
    int p = (rank + i) % n;
    CUmemGenericAllocationHandle h = mine;
    if (p != rank) {
      int pfd = -1;
      BCHECK(boot.recvFd(p, tag, &pfd));
      CUresult r = d.cuMemImportFromShareableHandle(&h, (void*)(uintptr_t)pfd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      ::close(pfd);
      if (r != CUDA_SUCCESS) BFAIL(ncclUnhandledCudaError, "importing rank %d's memory failed: %s", p, cuErrStr(r));
      seg->handle[p] = h;
    }
    BCU(d.cuMemMap(seg->vaBase + (size_t)p * size, size, 0, h, 0));
    seg->peer[p] = (char*)(seg->vaBase + (size_t)p * size);
  }
  CUmemAccessDesc ad{};
  ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  ad.location.id = cudaDev;
  ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  BCU(d.cuMemSetAccess(seg->vaBase, size * n, &ad, 1));
  if (localPtr) seg->peer[rank] = (char*)localPtr;  // adopted memory keeps its user-visible address
  BCHECK(boot.barrier());
  if (wantMc) BCHECK(setupMulticast(boot, cudaDev, tag + 1, seg));
  return ncclSuccess;
}

static ncclResult_t mapExchangeLegacy(Bootstrap& boot, int cudaDev, void* localPtr, size_t size, SymSeg* seg) {
  const int n = boot.nranks(), rank = boot.rank();
  seg->size = size;
  seg->nranks = n;
  seg->rank = rank;
  seg->legacy = true;
  struct Info { int pid; int dev; void* ptr; cudaIpcMemHandle_t h; } mine{}, all[kMaxRanks];
  mine.pid = (int)getpid();
  mine.dev = cudaDev;
  mine.ptr = localPtr;
  BCUDA(cudaIpcGetMemHandle(&mine.h, localPtr));
  BCHECK(boot.allGather(&mine, all, sizeof(Info)));
  for (int p = 0; p < n; p++) {
    if (p == rank) { seg->peer[p] = (char*)localPtr; continue; }
    if (all[p].pid == mine.pid) {
      if (all[p].dev != cudaDev) {
        cudaError_t e = cudaDeviceEnablePeerAccess(all[p].dev, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) BFAIL(ncclUnhandledCudaError, "peer access %d->%d refused: %s", cudaDev, all[p].dev, cudaGetErrorString(e));
        (void)cudaGetLastError();
      }
      seg->peer[p] = (char*)all[p].ptr;
    } else {
      void* q = nullptr;
      BCUDA(cudaIpcOpenMemHandle(&q, all[p].h, cudaIpcMemLazyEnablePeerAccess));
      seg->peer[p] = (char*)q;
      seg->legacyBase[p] = q;
    }
  }
  return boot.barrier();
}

static ncclResult_t agreeOnMode(Bootstrap& boot, int cudaDev, bool wantMc, bool* vmm, bool* mc, size_t* gran) {
  MemCaps caps;
  BCHECK(queryMemCaps(cudaDev, &caps));
  const Flags& fl = Flags::get();
  bool myVmm = caps.vmm && !fl.ipcLegacy && !failPoint("mem_no_vmm");
  bool myMc = myVmm && caps.multicast && wantMc && fl.nvlsEnable && boot.nranks() > 1 && !failPoint("mem_no_mc");
  BCHECK(allAgree(boot, myVmm, vmm));
  BCHECK(allAgree(boot, myMc, mc));
  *gran = caps.allocGran;
  if (*mc && caps.mcGran > *gran) *gran = caps.mcGran;
  return ncclSuccess;
}

ncclResult_t symAlloc(Bootstrap& boot, int cudaDev, size_t bytes, bool wantMc, uint32_t tag, SymSeg* seg) {
  *seg = SymSeg();
  bool vmm = false, mc = false;
  size_t gran = 2u << 20;
  BCHECK(agreeOnMode(boot, cudaDev, wantMc, &vmm, &mc, &gran));
  const size_t size = roundUp(bytes ? bytes : 1, gran);
  seg->ownsLocal = true;
  if (vmm) {
    const CuDrv& d = CuDrv::get();
    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = cudaDev;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUmemGenericAllocationHandle h;
    BCU(d.cuMemCreate(&h, size, &prop, 0));
    BCHECK(mapExchangeVmm(boot, cudaDev, h, nullptr, size, mc, tag, seg));
  } else {
    void* p = nullptr;
    BCUDA(cudaMalloc(&p, size));
    BCHECK(mapExchangeLegacy(boot, cudaDev, p, size, seg));
  }
  BINFO(SUB_MEM, "rank %d: symmetric segment of %zu bytes (%s%s)", boot.rank(), size, vmm ? "vmm" : "legacy ipc", seg->mc ? ", multicast" : "");
  return ncclSuccess;
}

ncclResult_t symAdopt(Bootstrap& boot, int cudaDev, void* localBase, size_t bytes, bool wantMc, uint32_t tag, SymSeg* seg) {
  *seg = SymSeg();
  LocalAlloc la;
  bool known = localAllocLookup(localBase, &la) && la.ptr == localBase && la.size >= bytes && la.vmm;
  bool vmm = false, mc = false, allKnown = false;
  size_t gran;
  BCHECK(agreeOnMode(boot, cudaDev, wantMc, &vmm, &mc, &gran));
  BCHECK(allAgree(boot, known, &allKnown));
  if (!vmm || !allKnown) BFAIL(ncclInvalidUsage, "buffer %p cannot be shared: it must come from ncclMemAlloc on every rank", localBase);
  // Sizes must match across ranks for a symmetric mapping.
  std::vector<size_t> sizes(boot.nranks());
  BCHECK(boot.allGather(&la.size, sizes.data(), sizeof(size_t)));
  for (size_t s : sizes) if (s != la.size) BFAIL(ncclInvalidUsage, "registered buffers differ in size across ranks (%zu vs %zu)", s, la.size);
  seg->ownsLocal = false;
  if (mc && (la.size % gran) != 0) mc = false;  // same on every rank since sizes are equal
  return mapExchangeVmm(boot, cudaDev, la.handle, localBase, la.size, mc, tag, seg);
}

ncclResult_t symFree(SymSeg* seg, int cudaDev) {
  if (seg->size == 0) return ncclSuccess;
  (void)cudaDev;
  if (seg->legacy) {
    for (int p = 0; p < seg->nranks; p++)
      if (seg->legacyBase[p]) cudaIpcCloseMemHandle(seg->legacyBase[p]);
    if (seg->ownsLocal && seg->peer[seg->rank]) cudaFree(seg->peer[seg->rank]);
    *seg = SymSeg();
    return ncclSuccess;
  }
  const CuDrv& d = CuDrv::get();
  if (seg->mcVa) {
    d.cuMemUnmap(seg->mcVa, seg->size);
    d.cuMemAddressFree(seg->mcVa, seg->size);
  }
  if (seg->mcHandle) {
    if (seg->mcBound) {
      CUdevice cuDev;
      if (d.cuDeviceGet(&cuDev, cudaDev) == CUDA_SUCCESS) d.cuMulticastUnbind(seg->mcHandle, cuDev, 0, seg->size);
    }
    d.cuMemRelease(seg->mcHandle);
  }
  if (seg->vaBase) {
    for (int p = 0; p < seg->nranks; p++) {
      d.cuMemUnmap(seg->vaBase + (size_t)p * seg->vaStride, seg->size);
      if (p != seg->rank && seg->handle[p]) d.cuMemRelease(seg->handle[p]);
    }
    d.cuMemAddressFree(seg->vaBase, seg->vaStride * seg->nranks);
  }
  if (seg->ownsLocal && seg->handle[seg->rank]) d.cuMemRelease(seg->handle[seg->rank]);
  *seg = SymSeg();
  return ncclSuccess;
}

// ---- ncclMemAlloc bookkeeping ----------------------------------------------------------------
static std::mutex gAllocMu;
static std::map<uintptr_t, LocalAlloc> gAllocs;

ncclResult_t localAllocExportable(void** ptr, size_t size) {
  if (!ptr) BFAIL(ncclInvalidArgument, "ncclMemAlloc: null pointer");
  int dev = 0;
  BCUDA(cudaGetDevice(&dev));
  BCUDA(cudaFree(0));
  MemCaps caps;
  BCHECK(queryMemCaps(dev, &caps));
  LocalAlloc la{};
  la.dev = dev;
  if (caps.vmm && !Flags::get().ipcLegacy) {
    const CuDrv& d = CuDrv::get();
    size_t gran = caps.allocGran;
    if (caps.multicast && caps.mcGran > gran) gran = caps.mcGran;
    la.size = roundUp(size ? size : 1, gran);
    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = dev;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    BCU(d.cuMemCreate(&la.handle, la.size, &prop, 0));
    CUdeviceptr va = 0;
    BCU(d.cuMemAddressReserve(&va, la.size, gran, 0, 0));
    BCU(d.cuMemMap(va, la.size, 0, la.handle, 0));
    // Readable and writable from this device and from every device that can reach it.
    int ndev = 0;
    cudaGetDeviceCount(&ndev);
    std::vector<CUmemAccessDesc> ads;
    for (int i = 0; i < ndev; i++) {
      int can = (i == dev);
      if (i != dev) cudaDeviceCanAccessPeer(&can, i, dev);
      if (!can) continue;
      CUmemAccessDesc ad{};
      ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      ad.location.id = i;
      ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      ads.push_back(ad);
    }
    BCU(d.cuMemSetAccess(va, la.size, ads.data(), ads.size()));
    la.ptr = (void*)va;
    la.vmm = true;
  } else {
    la.size = size;
    BCUDA(cudaMalloc(&la.ptr, size ? size : 1));
    la.vmm = false;
  }
  {
    std::lock_guard<std::mutex> lk(gAllocMu);
    gAllocs[(uintptr_t)la.ptr] = la;
  }
  *ptr = la.ptr;
  return ncclSuccess;
}

ncclResult_t localFreeExportable(void* ptr) {
  if (!ptr) return ncclSuccess;
  LocalAlloc la;
  {
    std::lock_guard<std::mutex> lk(gAllocMu);
    auto it = gAllocs.find((uintptr_t)ptr);
    if (it == gAllocs.end()) BFAIL(ncclInvalidArgument, "ncclMemFree: %p was not returned by ncclMemAlloc", ptr);
    la = it->second;
    gAllocs.erase(it);
  }
  if (la.vmm) {
    const CuDrv& d = CuDrv::get();
    BCU(d.cuMemUnmap((CUdeviceptr)la.ptr, la.size));
    BCU(d.cuMemRelease(la.handle));
    BCU(d.cuMemAddressFree((CUdeviceptr)la.ptr, la.size));
  } else {
    BCUDA(cudaFree(la.ptr));
  }
  return ncclSuccess;
}

bool localAllocLookup(const void* ptr, LocalAlloc* out) {
  std::lock_guard<std::mutex> lk(gAllocMu);
  auto it = gAllocs.upper_bound((uintptr_t)ptr);
  if (it == gAllocs.begin()) return false;
  --it;
  if ((uintptr_t)ptr >= it->first + it->second.size) return false;
  if (out) *out = it->second;
  return true;
}

}  // namespace b200
