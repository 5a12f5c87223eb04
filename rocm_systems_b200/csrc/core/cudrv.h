// CUDA driver entry points, fetched through the runtime so the library has no link-time
// dependency on libcuda (it must load on a build box that has no driver).
#pragma once

#include <cuda.h>

#include "common.h"

namespace b200 {

struct CuDrv {
  bool ok = false;
#define B200_DRV_FN(name) decltype(&::name) name = nullptr;
  B200_DRV_FN(cuGetErrorString)
  B200_DRV_FN(cuDeviceGet)
  B200_DRV_FN(cuDeviceGetAttribute)
  B200_DRV_FN(cuCtxGetDevice)
  B200_DRV_FN(cuMemCreate)
  B200_DRV_FN(cuMemRelease)
  B200_DRV_FN(cuMemAddressReserve)
  B200_DRV_FN(cuMemAddressFree)
  B200_DRV_FN(cuMemMap)
  B200_DRV_FN(cuMemUnmap)
  B200_DRV_FN(cuMemSetAccess)
  B200_DRV_FN(cuMemExportToShareableHandle)
  B200_DRV_FN(cuMemImportFromShareableHandle)
  B200_DRV_FN(cuMemGetAllocationGranularity)
  B200_DRV_FN(cuMemRetainAllocationHandle)
  B200_DRV_FN(cuMemGetAddressRange)
  B200_DRV_FN(cuMulticastCreate)
  B200_DRV_FN(cuMulticastAddDevice)
  B200_DRV_FN(cuMulticastBindMem)
  B200_DRV_FN(cuMulticastUnbind)
  B200_DRV_FN(cuMulticastGetGranularity)
  B200_DRV_FN(cuTensorMapEncodeTiled)
  B200_DRV_FN(cuPointerGetAttribute)
  B200_DRV_FN(cuStreamWriteValue32)  // optional: null on a driver without stream memory operations
#undef B200_DRV_FN
  static const CuDrv& get();  // loads once; `ok` is false when there is no driver
};

const char* cuErrStr(CUresult r);

#define BCU(call)                                                                          \
  do {                                                                                     \
    CUresult r__ = (call);                                                                 \
    if (r__ != CUDA_SUCCESS) {                                                             \
      ::b200::setLastError("%s:%d driver error '%s' from %s", ::b200::baseName(__FILE__), __LINE__,          \
                           ::b200::cuErrStr(r__), #call);                                  \
      BWARN("driver error '%s' from %s", ::b200::cuErrStr(r__), #call);                    \
      return ncclUnhandledCudaError;                                                       \
    }                                                                                      \
  } while (0)

}  // namespace b200
