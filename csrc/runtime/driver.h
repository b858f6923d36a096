// CUDA driver API loaded at run time with dlopen, so the runtime module imports on a
// machine without a GPU driver (it then reports zero devices) and carries no link-time
// dependency on libcuda.
#pragma once
#include <cuda.h>

#include <string>

namespace spike {

struct Driver {
  bool loaded = false;
  std::string load_error;
#define SPIKE_DRV(name) decltype(&::name) name = nullptr
  SPIKE_DRV(cuInit);
  SPIKE_DRV(cuDeviceGetCount);
  SPIKE_DRV(cuDeviceGet);
  SPIKE_DRV(cuDeviceGetName);
  SPIKE_DRV(cuDeviceGetAttribute);
  SPIKE_DRV(cuDeviceTotalMem_v2);
  SPIKE_DRV(cuDevicePrimaryCtxRetain);
  SPIKE_DRV(cuDevicePrimaryCtxRelease_v2);
  SPIKE_DRV(cuCtxSetCurrent);
  SPIKE_DRV(cuCtxSynchronize);
  SPIKE_DRV(cuMemAlloc_v2);
  SPIKE_DRV(cuMemFree_v2);
  SPIKE_DRV(cuMemcpyHtoD_v2);
  SPIKE_DRV(cuMemcpyDtoH_v2);
  SPIKE_DRV(cuMemcpyDtoDAsync_v2);
  SPIKE_DRV(cuMemcpyHtoDAsync_v2);
  SPIKE_DRV(cuMemcpyDtoHAsync_v2);
  SPIKE_DRV(cuMemsetD8_v2);
  SPIKE_DRV(cuModuleLoadData);
  SPIKE_DRV(cuModuleUnload);
  SPIKE_DRV(cuModuleGetFunction);
  SPIKE_DRV(cuFuncSetAttribute);
  SPIKE_DRV(cuLaunchKernel);
  SPIKE_DRV(cuStreamCreate);
  SPIKE_DRV(cuStreamDestroy_v2);
  SPIKE_DRV(cuStreamSynchronize);
  SPIKE_DRV(cuEventCreate);
  SPIKE_DRV(cuEventDestroy_v2);
  SPIKE_DRV(cuEventRecord);
  SPIKE_DRV(cuEventSynchronize);
  SPIKE_DRV(cuEventElapsedTime);
  SPIKE_DRV(cuGetErrorString);
  SPIKE_DRV(cuGetErrorName);
  SPIKE_DRV(cuTensorMapEncodeTiled);
  // virtual memory management + NVLink multicast objects (symmetric.cpp).  Optional: a driver without them
  // still loads, `vmm_loaded` / `multicast_loaded` say what is there.
  SPIKE_DRV(cuMemCreate);
  SPIKE_DRV(cuMemRelease);
  SPIKE_DRV(cuMemAddressReserve);
  SPIKE_DRV(cuMemAddressFree);
  SPIKE_DRV(cuMemMap);
  SPIKE_DRV(cuMemUnmap);
  SPIKE_DRV(cuMemSetAccess);
  SPIKE_DRV(cuMemGetAllocationGranularity);
  SPIKE_DRV(cuMemExportToShareableHandle);
  SPIKE_DRV(cuMemImportFromShareableHandle);
  SPIKE_DRV(cuMulticastCreate);
  SPIKE_DRV(cuMulticastAddDevice);
  SPIKE_DRV(cuMulticastBindMem);
  SPIKE_DRV(cuMulticastUnbind);
  SPIKE_DRV(cuMulticastGetGranularity);
#undef SPIKE_DRV
  bool vmm_loaded = false;
  bool multicast_loaded = false;
};

// Loads libcuda on first use; never throws (check `loaded`).
const Driver& driver();

// Throws CudaError with the failing call, the driver's error name and message.
void check(CUresult r, const char* what);
std::string cuda_error_string(CUresult r);

}  // namespace spike
