#include "driver.h"

#include <dlfcn.h>

#include <mutex>

#include "error.h"

namespace spike {

static Driver g_driver;
static std::once_flag g_once;

static void load() {
  void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) {
    const char* err = dlerror();
    g_driver.load_error = err ? err : "libcuda not found";
    return;
  }
  bool ok = true;
#define SPIKE_LOAD(name)                                                    \
  g_driver.name = reinterpret_cast<decltype(g_driver.name)>(dlsym(h, #name)); \
  if (!g_driver.name) {                                                     \
    ok = false;                                                             \
    g_driver.load_error += std::string(" missing ") + #name;                \
  }
  SPIKE_LOAD(cuInit);
  SPIKE_LOAD(cuDeviceGetCount);
  SPIKE_LOAD(cuDeviceGet);
  SPIKE_LOAD(cuDeviceGetName);
  SPIKE_LOAD(cuDeviceGetAttribute);
  SPIKE_LOAD(cuDeviceTotalMem_v2);
  SPIKE_LOAD(cuDevicePrimaryCtxRetain);
  SPIKE_LOAD(cuDevicePrimaryCtxRelease_v2);
  SPIKE_LOAD(cuCtxSetCurrent);
  SPIKE_LOAD(cuCtxSynchronize);
  SPIKE_LOAD(cuMemAlloc_v2);
  SPIKE_LOAD(cuMemFree_v2);
  SPIKE_LOAD(cuMemcpyHtoD_v2);
  SPIKE_LOAD(cuMemcpyDtoH_v2);
  SPIKE_LOAD(cuMemcpyDtoDAsync_v2);
  SPIKE_LOAD(cuMemcpyHtoDAsync_v2);
  SPIKE_LOAD(cuMemcpyDtoHAsync_v2);
  SPIKE_LOAD(cuMemsetD8_v2);
  SPIKE_LOAD(cuModuleLoadData);
  SPIKE_LOAD(cuModuleUnload);
  SPIKE_LOAD(cuModuleGetFunction);
  SPIKE_LOAD(cuFuncSetAttribute);
  SPIKE_LOAD(cuLaunchKernel);
  SPIKE_LOAD(cuStreamCreate);
  SPIKE_LOAD(cuStreamDestroy_v2);
  SPIKE_LOAD(cuStreamSynchronize);
  SPIKE_LOAD(cuEventCreate);
  SPIKE_LOAD(cuEventDestroy_v2);
  SPIKE_LOAD(cuEventRecord);
  SPIKE_LOAD(cuEventSynchronize);
  SPIKE_LOAD(cuEventElapsedTime);
  SPIKE_LOAD(cuGetErrorString);
  SPIKE_LOAD(cuGetErrorName);
  SPIKE_LOAD(cuTensorMapEncodeTiled);
#undef SPIKE_LOAD
  g_driver.loaded = ok;
  bool vmm = true, mc = true;
#define SPIKE_OPT(flag, name)                                                 \
  g_driver.name = reinterpret_cast<decltype(g_driver.name)>(dlsym(h, #name)); \
  if (!g_driver.name) flag = false;
  SPIKE_OPT(vmm, cuMemCreate);
  SPIKE_OPT(vmm, cuMemRelease);
  SPIKE_OPT(vmm, cuMemAddressReserve);
  SPIKE_OPT(vmm, cuMemAddressFree);
  SPIKE_OPT(vmm, cuMemMap);
  SPIKE_OPT(vmm, cuMemUnmap);
  SPIKE_OPT(vmm, cuMemSetAccess);
  SPIKE_OPT(vmm, cuMemGetAllocationGranularity);
  SPIKE_OPT(vmm, cuMemExportToShareableHandle);
  SPIKE_OPT(vmm, cuMemImportFromShareableHandle);
  SPIKE_OPT(mc, cuMulticastCreate);
  SPIKE_OPT(mc, cuMulticastAddDevice);
  SPIKE_OPT(mc, cuMulticastBindMem);
  SPIKE_OPT(mc, cuMulticastUnbind);
  SPIKE_OPT(mc, cuMulticastGetGranularity);
#undef SPIKE_OPT
  g_driver.vmm_loaded = ok && vmm;
  g_driver.multicast_loaded = ok && vmm && mc;
}

const Driver& driver() {
  std::call_once(g_once, load);
  return g_driver;
}

std::string cuda_error_string(CUresult r) {
  const Driver& d = driver();
  const char* name = nullptr;
  const char* msg = nullptr;
  if (d.loaded) {
    d.cuGetErrorName(r, &name);
    d.cuGetErrorString(r, &msg);
  }
  return std::string(name ? name : "CUDA_ERROR_UNKNOWN") + " (" + std::to_string(static_cast<int>(r)) + "): " +
         (msg ? msg : "no description");
}

void check(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) throw CudaError(static_cast<int>(r), std::string(what) + " failed: " + cuda_error_string(r));
}

}  // namespace spike
