#include "cudrv.h"

#include <mutex>

namespace b200 {

static CuDrv gDrv;
static std::once_flag gDrvOnce;

template <typename F>
static bool loadOne(const char* name, F* out) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
    (void)cudaGetLastError();
    *out = nullptr;
    return false;
  }
  *out = reinterpret_cast<F>(fn);
  return true;
}

const CuDrv& CuDrv::get() {
  std::call_once(gDrvOnce, [] {
    bool all = true;
#define B200_DRV_LOAD(name) all = loadOne(#name, &gDrv.name) && all;
    B200_DRV_LOAD(cuGetErrorString)
    B200_DRV_LOAD(cuDeviceGet)
    B200_DRV_LOAD(cuDeviceGetAttribute)
    B200_DRV_LOAD(cuCtxGetDevice)
    B200_DRV_LOAD(cuMemCreate)
    B200_DRV_LOAD(cuMemRelease)
    B200_DRV_LOAD(cuMemAddressReserve)
    B200_DRV_LOAD(cuMemAddressFree)
    B200_DRV_LOAD(cuMemMap)
    B200_DRV_LOAD(cuMemUnmap)
    B200_DRV_LOAD(cuMemSetAccess)
    B200_DRV_LOAD(cuMemExportToShareableHandle)
    B200_DRV_LOAD(cuMemImportFromShareableHandle)
    B200_DRV_LOAD(cuMemGetAllocationGranularity)
    B200_DRV_LOAD(cuMemRetainAllocationHandle)
    B200_DRV_LOAD(cuMemGetAddressRange)
    B200_DRV_LOAD(cuMulticastCreate)
    B200_DRV_LOAD(cuMulticastAddDevice)
    B200_DRV_LOAD(cuMulticastBindMem)
    B200_DRV_LOAD(cuMulticastUnbind)
    B200_DRV_LOAD(cuMulticastGetGranularity)
    B200_DRV_LOAD(cuTensorMapEncodeTiled)
    B200_DRV_LOAD(cuPointerGetAttribute)
#undef B200_DRV_LOAD
    loadOne("cuStreamWriteValue32", &gDrv.cuStreamWriteValue32);  // optional
    gDrv.ok = all;
    if (!all) BINFO(SUB_INIT, "CUDA driver entry points unavailable (no driver on this machine?)");
  });
  return gDrv;
}

const char* cuErrStr(CUresult r) {
  const CuDrv& d = CuDrv::get();
  const char* s = nullptr;
  if (d.cuGetErrorString && d.cuGetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "unknown driver error";
}

}  // namespace b200
