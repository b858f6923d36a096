// A stand-in for the CUDA driver library, for testing the C++ device runtime on a machine without a GPU.
// Device memory is host memory, modules hold no code, launches and copies are appended to a log.  Built by the
// tests as libcuda.so.1 and put first on the library path of a child process.
//
// Controlled through the environment of that process:
//   FAKE_CUDA_DEVICES=N           number of devices reported (default 1)
//   FAKE_CUDA_LOG=path            one line per call worth checking: launches, module loads, frees
//   FAKE_CUDA_FAIL=name:code[:n]  the n-th call (default: every call) of driver function `name` returns `code`
//                                 (host-side failure injection: an error code from a fake of the failing call)
//   FAKE_CUDA_EVENT_MS=x          elapsed time reported between any two events (default 0.25)
#include <cuda.h>
#include <sys/mman.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <string>

namespace {
std::mutex g_mu;
std::map<std::string, int> g_calls;
std::set<void*> g_live;                 // device allocations (host pointers)
struct Module { int id; };
struct Function { std::string name; int smem = 0; };
int g_next_module = 1;
size_t g_bytes_live = 0;
std::map<void*, size_t> g_sizes;

int devices() {
  const char* e = std::getenv("FAKE_CUDA_DEVICES");
  return e ? std::atoi(e) : 1;
}

void log_line(const std::string& s) {
  const char* p = std::getenv("FAKE_CUDA_LOG");
  if (!p) return;
  if (FILE* f = std::fopen(p, "a")) {
    std::fputs(s.c_str(), f);
    std::fputc('\n', f);
    std::fclose(f);
  }
}

// returns the injected error for this call, or CUDA_SUCCESS
CUresult enter(const char* name) {
  std::lock_guard<std::mutex> lk(g_mu);
  const int n = ++g_calls[name];
  const char* e = std::getenv("FAKE_CUDA_FAIL");
  if (!e) return CUDA_SUCCESS;
  std::string spec = e;
  const size_t c1 = spec.find(':');
  if (c1 == std::string::npos || spec.substr(0, c1) != name) return CUDA_SUCCESS;
  const size_t c2 = spec.find(':', c1 + 1);
  const int code = std::atoi(spec.substr(c1 + 1, c2 == std::string::npos ? std::string::npos : c2 - c1 - 1).c_str());
  if (c2 != std::string::npos && std::atoi(spec.substr(c2 + 1).c_str()) != n) return CUDA_SUCCESS;
  return static_cast<CUresult>(code);
}

bool inside_live(const void* p, size_t n) {
  for (void* base : g_live) {
    const char* b = static_cast<const char*>(base);
    if (static_cast<const char*>(p) >= b && static_cast<const char*>(p) + n <= b + g_sizes[base]) return true;
  }
  return false;
}
}  // namespace

#define FAKE_ENTER(name)                      \
  do {                                        \
    CUresult _r = enter(name);                \
    if (_r != CUDA_SUCCESS) return _r;        \
  } while (0)

extern "C" {

CUresult cuInit(unsigned) { FAKE_ENTER("cuInit"); return CUDA_SUCCESS; }
CUresult cuDeviceGetCount(int* n) { FAKE_ENTER("cuDeviceGetCount"); *n = devices(); return CUDA_SUCCESS; }
CUresult cuDeviceGet(CUdevice* d, int ordinal) {
  FAKE_ENTER("cuDeviceGet");
  if (ordinal < 0 || ordinal >= devices()) return CUDA_ERROR_INVALID_DEVICE;
  *d = ordinal;
  return CUDA_SUCCESS;
}
CUresult cuDeviceGetName(char* name, int len, CUdevice d) {
  FAKE_ENTER("cuDeviceGetName");
  std::snprintf(name, size_t(len), "Fake B200 #%d", int(d));
  return CUDA_SUCCESS;
}
CUresult cuDeviceGetAttribute(int* v, CUdevice_attribute a, CUdevice) {
  FAKE_ENTER("cuDeviceGetAttribute");
  switch (a) {
    case CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT: *v = 148; break;
    case CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR: *v = 10; break;
    case CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR: *v = 0; break;
    case CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN: *v = 232448; break;
    case CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED: *v = 1; break;
    case CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED: *v = 1; break;
    case CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED: *v = std::getenv("FAKE_CUDA_NO_MULTICAST") ? 0 : 1; break;
    default: *v = 0; break;
  }
  return CUDA_SUCCESS;
}
CUresult cuDeviceTotalMem_v2(size_t* n, CUdevice) { FAKE_ENTER("cuDeviceTotalMem_v2"); *n = size_t(180) << 30; return CUDA_SUCCESS; }
CUresult cuDevicePrimaryCtxRetain(CUcontext* c, CUdevice d) {
  FAKE_ENTER("cuDevicePrimaryCtxRetain");
  *c = reinterpret_cast<CUcontext>(uintptr_t(0x1000 + d));
  return CUDA_SUCCESS;
}
CUresult cuDevicePrimaryCtxRelease_v2(CUdevice) { FAKE_ENTER("cuDevicePrimaryCtxRelease_v2"); log_line("ctx_release"); return CUDA_SUCCESS; }
CUresult cuCtxSetCurrent(CUcontext) { FAKE_ENTER("cuCtxSetCurrent"); return CUDA_SUCCESS; }
CUresult cuCtxSynchronize() { FAKE_ENTER("cuCtxSynchronize"); return CUDA_SUCCESS; }

CUresult cuMemAlloc_v2(CUdeviceptr* p, size_t n) {
  FAKE_ENTER("cuMemAlloc_v2");
  void* h = std::calloc(1, n ? n : 1);
  if (!h) return CUDA_ERROR_OUT_OF_MEMORY;
  std::lock_guard<std::mutex> lk(g_mu);
  g_live.insert(h);
  g_sizes[h] = n;
  g_bytes_live += n;
  *p = reinterpret_cast<CUdeviceptr>(h);
  return CUDA_SUCCESS;
}
CUresult cuMemFree_v2(CUdeviceptr p) {
  FAKE_ENTER("cuMemFree_v2");
  void* h = reinterpret_cast<void*>(p);
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_live.count(h)) {
      log_line("bad_free");
      return CUDA_ERROR_INVALID_VALUE;
    }
    g_live.erase(h);
    g_bytes_live -= g_sizes[h];
    g_sizes.erase(h);
  }
  std::free(h);
  log_line("free live_bytes=" + std::to_string(g_bytes_live));
  return CUDA_SUCCESS;
}
static CUresult copy_checked(const char* what, void* dst, const void* src, size_t n, const void* dev, bool log) {
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!inside_live(dev, n)) {
      log_line(std::string("out_of_bounds ") + what);
      return CUDA_ERROR_INVALID_VALUE;
    }
  }
  std::memcpy(dst, src, n);
  if (log) log_line(std::string(what) + " bytes=" + std::to_string(n));
  return CUDA_SUCCESS;
}
CUresult cuMemcpyHtoD_v2(CUdeviceptr d, const void* s, size_t n) {
  FAKE_ENTER("cuMemcpyHtoD_v2");
  return copy_checked("h2d", reinterpret_cast<void*>(d), s, n, reinterpret_cast<void*>(d), false);
}
CUresult cuMemcpyDtoH_v2(void* d, CUdeviceptr s, size_t n) {
  FAKE_ENTER("cuMemcpyDtoH_v2");
  return copy_checked("d2h", d, reinterpret_cast<void*>(s), n, reinterpret_cast<void*>(s), false);
}
CUresult cuMemcpyHtoDAsync_v2(CUdeviceptr d, const void* s, size_t n, CUstream) {
  FAKE_ENTER("cuMemcpyHtoDAsync_v2");
  return copy_checked("h2d_async", reinterpret_cast<void*>(d), s, n, reinterpret_cast<void*>(d), false);
}
CUresult cuMemcpyDtoHAsync_v2(void* d, CUdeviceptr s, size_t n, CUstream) {
  FAKE_ENTER("cuMemcpyDtoHAsync_v2");
  return copy_checked("d2h_async", d, reinterpret_cast<void*>(s), n, reinterpret_cast<void*>(s), false);
}
CUresult cuMemcpyDtoDAsync_v2(CUdeviceptr d, CUdeviceptr s, size_t n, CUstream) {
  FAKE_ENTER("cuMemcpyDtoDAsync_v2");
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!inside_live(reinterpret_cast<void*>(s), n)) return CUDA_ERROR_INVALID_VALUE;
  }
  return copy_checked("d2d", reinterpret_cast<void*>(d), reinterpret_cast<void*>(s), n, reinterpret_cast<void*>(d), true);
}
CUresult cuMemsetD8_v2(CUdeviceptr d, unsigned char v, size_t n) {
  FAKE_ENTER("cuMemsetD8_v2");
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!inside_live(reinterpret_cast<void*>(d), n)) return CUDA_ERROR_INVALID_VALUE;
  }
  std::memset(reinterpret_cast<void*>(d), v, n);
  return CUDA_SUCCESS;
}

CUresult cuModuleLoadData(CUmodule* m, const void* image) {
  FAKE_ENTER("cuModuleLoadData");
  if (!image) return CUDA_ERROR_INVALID_IMAGE;
  auto* mod = new Module{g_next_module++};
  *m = reinterpret_cast<CUmodule>(mod);
  log_line("module_load id=" + std::to_string(mod->id));
  return CUDA_SUCCESS;
}
CUresult cuModuleUnload(CUmodule m) {
  FAKE_ENTER("cuModuleUnload");
  auto* mod = reinterpret_cast<Module*>(m);
  log_line("module_unload id=" + std::to_string(mod->id));
  delete mod;
  return CUDA_SUCCESS;
}
CUresult cuModuleGetFunction(CUfunction* f, CUmodule, const char* name) {
  FAKE_ENTER("cuModuleGetFunction");
  if (std::strncmp(name, "missing_", 8) == 0) return CUDA_ERROR_NOT_FOUND;
  *f = reinterpret_cast<CUfunction>(new Function{name});        // lives as long as the process: functions are never freed
  return CUDA_SUCCESS;
}
CUresult cuFuncSetAttribute(CUfunction f, CUfunction_attribute a, int v) {
  FAKE_ENTER("cuFuncSetAttribute");
  if (a == CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES) {
    if (v > 232448) return CUDA_ERROR_INVALID_VALUE;
    reinterpret_cast<Function*>(f)->smem = v;
  }
  return CUDA_SUCCESS;
}
CUresult cuLaunchKernel(CUfunction f, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by, unsigned bz,
                        unsigned smem, CUstream, void** params, void**) {
  FAKE_ENTER("cuLaunchKernel");
  auto* fn = reinterpret_cast<Function*>(f);
  if (gx == 0 || gy == 0 || gz == 0 || bx * by * bz == 0 || bx * by * bz > 1024) return CUDA_ERROR_INVALID_VALUE;
  if (smem > 49152u && int(smem) > fn->smem) return CUDA_ERROR_INVALID_VALUE;   // opt-in shared memory not requested
  char buf[256];
  std::snprintf(buf, sizeof buf, "launch %s grid=%u,%u,%u block=%u,%u,%u smem=%u params=%s", fn->name.c_str(), gx, gy,
                gz, bx, by, bz, smem, params ? "yes" : "no");
  log_line(buf);
  return CUDA_SUCCESS;
}

CUresult cuStreamCreate(CUstream* s, unsigned) { FAKE_ENTER("cuStreamCreate"); *s = reinterpret_cast<CUstream>(uintptr_t(0x2000)); return CUDA_SUCCESS; }
CUresult cuStreamDestroy_v2(CUstream) { FAKE_ENTER("cuStreamDestroy_v2"); return CUDA_SUCCESS; }
CUresult cuStreamSynchronize(CUstream) { FAKE_ENTER("cuStreamSynchronize"); return CUDA_SUCCESS; }
CUresult cuEventCreate(CUevent* e, unsigned) { FAKE_ENTER("cuEventCreate"); *e = reinterpret_cast<CUevent>(new int(0)); return CUDA_SUCCESS; }
CUresult cuEventDestroy_v2(CUevent e) { FAKE_ENTER("cuEventDestroy_v2"); delete reinterpret_cast<int*>(e); return CUDA_SUCCESS; }
CUresult cuEventRecord(CUevent, CUstream) { FAKE_ENTER("cuEventRecord"); return CUDA_SUCCESS; }
CUresult cuEventSynchronize(CUevent) { FAKE_ENTER("cuEventSynchronize"); return CUDA_SUCCESS; }
CUresult cuEventElapsedTime(float* ms, CUevent, CUevent) {
  FAKE_ENTER("cuEventElapsedTime");
  const char* e = std::getenv("FAKE_CUDA_EVENT_MS");
  *ms = e ? float(std::atof(e)) : 0.25f;
  return CUDA_SUCCESS;
}
CUresult cuGetErrorString(CUresult r, const char** s) {
  switch (r) {
    case CUDA_ERROR_INVALID_VALUE: *s = "invalid argument"; break;
    case CUDA_ERROR_OUT_OF_MEMORY: *s = "out of memory"; break;
    case CUDA_ERROR_LAUNCH_FAILED: *s = "unspecified launch failure"; break;
    case CUDA_ERROR_ILLEGAL_ADDRESS: *s = "an illegal memory access was encountered"; break;
    case CUDA_ERROR_LAUNCH_TIMEOUT: *s = "the launch timed out and was terminated"; break;
    default: *s = "fake driver error"; break;
  }
  return CUDA_SUCCESS;
}
CUresult cuGetErrorName(CUresult r, const char** s) {
  switch (r) {
    case CUDA_ERROR_INVALID_VALUE: *s = "CUDA_ERROR_INVALID_VALUE"; break;
    case CUDA_ERROR_OUT_OF_MEMORY: *s = "CUDA_ERROR_OUT_OF_MEMORY"; break;
    case CUDA_ERROR_LAUNCH_FAILED: *s = "CUDA_ERROR_LAUNCH_FAILED"; break;
    case CUDA_ERROR_ILLEGAL_ADDRESS: *s = "CUDA_ERROR_ILLEGAL_ADDRESS"; break;
    case CUDA_ERROR_LAUNCH_TIMEOUT: *s = "CUDA_ERROR_LAUNCH_TIMEOUT"; break;
    case CUDA_ERROR_INVALID_DEVICE: *s = "CUDA_ERROR_INVALID_DEVICE"; break;
    case CUDA_ERROR_NOT_FOUND: *s = "CUDA_ERROR_NOT_FOUND"; break;
    default: *s = "CUDA_ERROR_FAKE"; break;
  }
  return CUDA_SUCCESS;
}
CUresult cuTensorMapEncodeTiled(CUtensorMap* map, CUtensorMapDataType, cuuint32_t rank, void* addr, const cuuint64_t*,
                                const cuuint64_t* strides, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) {
  FAKE_ENTER("cuTensorMapEncodeTiled");
  // the checks the real encoder makes and the runtime relies on: base address and strides multiples of 16 bytes
  if (reinterpret_cast<uintptr_t>(addr) % 16) return CUDA_ERROR_INVALID_VALUE;
  for (cuuint32_t i = 0; i + 1 < rank; ++i)
    if (strides[i] % 16) return CUDA_ERROR_INVALID_VALUE;
  std::memset(map, 0, sizeof(*map));
  log_line("tensor_map rank=" + std::to_string(rank));
  return CUDA_SUCCESS;
}

}  // extern "C"

// ---- virtual memory management: an allocation is an anonymous file (memfd), a mapping is an mmap of it at a reserved
// address, a shareable handle is a duplicate of the descriptor.  Two mappings of one allocation alias, in one process or
// in two, as peer mappings of device memory do.  A multicast object is a file of its own; binding only checks the
// protocol (every device added before the first bind), since there is no switch to reduce in.
namespace {
constexpr size_t kGranularity = 2u << 20;
struct Alloc {
  int fd = -1;
  size_t size = 0;
  bool multicast = false;
  unsigned want_devices = 0, added = 0, bound = 0;
  int refs = 1;
};
std::map<CUmemGenericAllocationHandle, Alloc*> g_allocs;
CUmemGenericAllocationHandle g_next_handle = 0x5000;
std::map<void*, size_t> g_reserved;      // address ranges from cuMemAddressReserve
std::map<void*, size_t> g_mapped;        // ranges currently backed by an allocation

Alloc* find_alloc(CUmemGenericAllocationHandle h) {
  auto it = g_allocs.find(h);
  return it == g_allocs.end() ? nullptr : it->second;
}
CUmemGenericAllocationHandle add_alloc(Alloc* a) {
  g_allocs[g_next_handle] = a;
  return g_next_handle++;
}
}  // namespace

extern "C" {
CUresult cuMemGetAllocationGranularity(size_t* g, const CUmemAllocationProp* prop, CUmemAllocationGranularity_flags) {
  FAKE_ENTER("cuMemGetAllocationGranularity");
  if (prop->location.id < 0 || prop->location.id >= devices()) return CUDA_ERROR_INVALID_DEVICE;
  *g = kGranularity;
  return CUDA_SUCCESS;
}
CUresult cuMulticastGetGranularity(size_t* g, const CUmulticastObjectProp*, CUmulticastGranularity_flags) {
  FAKE_ENTER("cuMulticastGetGranularity");
  *g = kGranularity;
  return CUDA_SUCCESS;
}
CUresult cuMemCreate(CUmemGenericAllocationHandle* h, size_t size, const CUmemAllocationProp* prop, unsigned long long) {
  FAKE_ENTER("cuMemCreate");
  if (size == 0 || size % kGranularity) return CUDA_ERROR_INVALID_VALUE;
  if (prop->requestedHandleTypes != CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) return CUDA_ERROR_NOT_SUPPORTED;
  int fd = memfd_create("fake_cuda_alloc", 0);
  if (fd < 0 || ftruncate(fd, off_t(size)) != 0) return CUDA_ERROR_OUT_OF_MEMORY;
  std::lock_guard<std::mutex> lk(g_mu);
  auto* a = new Alloc;
  a->fd = fd;
  a->size = size;
  *h = add_alloc(a);
  log_line("mem_create bytes=" + std::to_string(size));
  return CUDA_SUCCESS;
}
CUresult cuMemRelease(CUmemGenericAllocationHandle h) {
  FAKE_ENTER("cuMemRelease");
  std::lock_guard<std::mutex> lk(g_mu);
  Alloc* a = find_alloc(h);
  if (!a) {
    log_line("bad_release");
    return CUDA_ERROR_INVALID_VALUE;
  }
  g_allocs.erase(h);
  if (--a->refs == 0) {
    close(a->fd);
    delete a;
  }
  log_line("mem_release live_handles=" + std::to_string(g_allocs.size()));
  return CUDA_SUCCESS;
}
CUresult cuMemAddressReserve(CUdeviceptr* va, size_t size, size_t align, CUdeviceptr, unsigned long long) {
  FAKE_ENTER("cuMemAddressReserve");
  if (size == 0 || size % kGranularity || (align && align % kGranularity)) return CUDA_ERROR_INVALID_VALUE;
  // over-reserve to align to the granularity, as device addresses are
  void* p = mmap(nullptr, size + kGranularity, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  if (p == MAP_FAILED) return CUDA_ERROR_OUT_OF_MEMORY;
  uintptr_t a = (reinterpret_cast<uintptr_t>(p) + kGranularity - 1) & ~(uintptr_t(kGranularity) - 1);
  std::lock_guard<std::mutex> lk(g_mu);
  g_reserved[reinterpret_cast<void*>(a)] = size;
  *va = CUdeviceptr(a);
  return CUDA_SUCCESS;
}
CUresult cuMemAddressFree(CUdeviceptr va, size_t size) {
  FAKE_ENTER("cuMemAddressFree");
  std::lock_guard<std::mutex> lk(g_mu);
  void* p = reinterpret_cast<void*>(va);
  auto it = g_reserved.find(p);
  if (it == g_reserved.end() || it->second != size) {
    log_line("bad_address_free");
    return CUDA_ERROR_INVALID_VALUE;
  }
  if (g_mapped.count(p)) {
    log_line("address_free_while_mapped");
    return CUDA_ERROR_INVALID_VALUE;
  }
  g_reserved.erase(it);
  munmap(p, size);
  return CUDA_SUCCESS;
}
CUresult cuMemMap(CUdeviceptr va, size_t size, size_t offset, CUmemGenericAllocationHandle h, unsigned long long) {
  FAKE_ENTER("cuMemMap");
  std::lock_guard<std::mutex> lk(g_mu);
  void* p = reinterpret_cast<void*>(va);
  Alloc* a = find_alloc(h);
  auto it = g_reserved.find(p);
  if (!a || it == g_reserved.end() || it->second != size || offset != 0 || size > a->size || g_mapped.count(p))
    return CUDA_ERROR_INVALID_VALUE;
  // not accessible until cuMemSetAccess, like the real thing
  if (mmap(p, size, PROT_NONE, MAP_SHARED | MAP_FIXED, a->fd, 0) == MAP_FAILED) return CUDA_ERROR_OUT_OF_MEMORY;
  g_mapped[p] = size;
  return CUDA_SUCCESS;
}
CUresult cuMemSetAccess(CUdeviceptr va, size_t size, const CUmemAccessDesc* desc, size_t count) {
  FAKE_ENTER("cuMemSetAccess");
  std::lock_guard<std::mutex> lk(g_mu);
  void* p = reinterpret_cast<void*>(va);
  if (!g_mapped.count(p) || g_mapped[p] != size || count < 1 || desc[0].flags != CU_MEM_ACCESS_FLAGS_PROT_READWRITE)
    return CUDA_ERROR_INVALID_VALUE;
  if (mprotect(p, size, PROT_READ | PROT_WRITE) != 0) return CUDA_ERROR_INVALID_VALUE;
  g_live.insert(p);               // plain copies and memsets may now touch it
  g_sizes[p] = size;
  return CUDA_SUCCESS;
}
CUresult cuMemUnmap(CUdeviceptr va, size_t size) {
  FAKE_ENTER("cuMemUnmap");
  std::lock_guard<std::mutex> lk(g_mu);
  void* p = reinterpret_cast<void*>(va);
  if (!g_mapped.count(p) || g_mapped[p] != size) {
    log_line("bad_unmap");
    return CUDA_ERROR_INVALID_VALUE;
  }
  g_mapped.erase(p);
  g_live.erase(p);
  g_sizes.erase(p);
  // back to a bare reservation
  mmap(p, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0);
  return CUDA_SUCCESS;
}
CUresult cuMemExportToShareableHandle(void* out, CUmemGenericAllocationHandle h, CUmemAllocationHandleType t,
                                      unsigned long long) {
  FAKE_ENTER("cuMemExportToShareableHandle");
  std::lock_guard<std::mutex> lk(g_mu);
  Alloc* a = find_alloc(h);
  if (!a || t != CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) return CUDA_ERROR_INVALID_VALUE;
  const int fd = dup(a->fd);
  if (fd < 0) return CUDA_ERROR_OUT_OF_MEMORY;
  *static_cast<int*>(out) = fd;
  return CUDA_SUCCESS;
}
CUresult cuMemImportFromShareableHandle(CUmemGenericAllocationHandle* h, void* os_handle, CUmemAllocationHandleType t) {
  FAKE_ENTER("cuMemImportFromShareableHandle");
  if (t != CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) return CUDA_ERROR_INVALID_VALUE;
  const int fd = dup(int(reinterpret_cast<intptr_t>(os_handle)));     // the caller keeps and closes its descriptor
  if (fd < 0) return CUDA_ERROR_INVALID_VALUE;
  const off_t size = lseek(fd, 0, SEEK_END);
  if (size <= 0) {
    close(fd);
    return CUDA_ERROR_INVALID_VALUE;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  auto* a = new Alloc;
  a->fd = fd;
  a->size = size_t(size);
  *h = add_alloc(a);
  return CUDA_SUCCESS;
}
CUresult cuMulticastCreate(CUmemGenericAllocationHandle* h, const CUmulticastObjectProp* prop) {
  FAKE_ENTER("cuMulticastCreate");
  if (prop->numDevices < 1 || prop->size == 0 || prop->size % kGranularity) return CUDA_ERROR_INVALID_VALUE;
  int fd = memfd_create("fake_cuda_multicast", 0);
  if (fd < 0 || ftruncate(fd, off_t(prop->size)) != 0) return CUDA_ERROR_OUT_OF_MEMORY;
  std::lock_guard<std::mutex> lk(g_mu);
  auto* a = new Alloc;
  a->fd = fd;
  a->size = prop->size;
  a->multicast = true;
  a->want_devices = prop->numDevices;
  *h = add_alloc(a);
  log_line("multicast_create devices=" + std::to_string(prop->numDevices));
  return CUDA_SUCCESS;
}
CUresult cuMulticastAddDevice(CUmemGenericAllocationHandle h, CUdevice) {
  FAKE_ENTER("cuMulticastAddDevice");
  std::lock_guard<std::mutex> lk(g_mu);
  Alloc* a = find_alloc(h);
  if (!a) return CUDA_ERROR_INVALID_VALUE;
  ++a->added;
  log_line("multicast_add_device");
  return CUDA_SUCCESS;
}
CUresult cuMulticastBindMem(CUmemGenericAllocationHandle mc, size_t mc_off, CUmemGenericAllocationHandle mem, size_t off,
                            size_t size, unsigned long long) {
  FAKE_ENTER("cuMulticastBindMem");
  std::lock_guard<std::mutex> lk(g_mu);
  Alloc* a = find_alloc(mc);
  Alloc* m = find_alloc(mem);
  if (!a || !m || mc_off || off || size > a->size || size > m->size) return CUDA_ERROR_INVALID_VALUE;
  ++a->bound;
  log_line("multicast_bind");
  return CUDA_SUCCESS;
}
CUresult cuMulticastUnbind(CUmemGenericAllocationHandle mc, CUdevice, size_t, size_t) {
  FAKE_ENTER("cuMulticastUnbind");
  std::lock_guard<std::mutex> lk(g_mu);
  Alloc* a = find_alloc(mc);
  if (!a || a->bound == 0) {
    log_line("bad_unbind");
    return CUDA_ERROR_INVALID_VALUE;
  }
  --a->bound;
  log_line("multicast_unbind");
  return CUDA_SUCCESS;
}
}  // extern "C"
