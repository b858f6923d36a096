#include "symmetric.h"

#include <unistd.h>

#include <algorithm>

#include "driver.h"
#include "error.h"

namespace spike {

namespace {

CUmemAllocationProp alloc_prop(int ordinal) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = ordinal;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

size_t round_up(size_t v, size_t g) { return g ? (v + g - 1) / g * g : v; }

void ensure_context(const Driver& d, int ordinal, CUdevice* dev) {
  check(d.cuInit(0), "cuInit");
  check(d.cuDeviceGet(dev, ordinal), "cuDeviceGet");
  // the primary context is the one the CUDA runtime API (and torch) uses; retaining it is reference counted
  CUcontext ctx = nullptr;
  check(d.cuDevicePrimaryCtxRetain(&ctx, *dev), "cuDevicePrimaryCtxRetain");
  check(d.cuCtxSetCurrent(ctx), "cuCtxSetCurrent");
}

}  // namespace

bool SymmetricBuffer::supported(int device_ordinal) {
  const Driver& d = driver();
  if (!d.loaded || !d.vmm_loaded) return false;
  if (d.cuInit(0) != CUDA_SUCCESS) return false;
  CUdevice dev;
  if (d.cuDeviceGet(&dev, device_ordinal) != CUDA_SUCCESS) return false;
  int vmm = 0, fd = 0;
  d.cuDeviceGetAttribute(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev);
  d.cuDeviceGetAttribute(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
  return vmm && fd;
}

bool SymmetricBuffer::multicast_supported(int device_ordinal) {
  const Driver& d = driver();
  if (!supported(device_ordinal) || !d.multicast_loaded) return false;
  CUdevice dev;
  if (d.cuDeviceGet(&dev, device_ordinal) != CUDA_SUCCESS) return false;
  int mc = 0;
  d.cuDeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
  return mc != 0;
}

SymmetricBuffer::SymmetricBuffer(int device_ordinal, size_t bytes) : ordinal_(device_ordinal) {
  const Driver& d = driver();
  if (!d.loaded) throw SpikeRuntimeError("CUDA driver library could not be loaded: " + d.load_error);
  if (!d.vmm_loaded) throw SpikeRuntimeError("this CUDA driver has no virtual memory management API");
  if (bytes == 0) throw SpikeError("symmetric buffer of zero bytes");
  ensure_context(d, device_ordinal, &device_);
  CUmemAllocationProp prop = alloc_prop(ordinal_);
  size_t g = 0;
  check(d.cuMemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  if (d.multicast_loaded && multicast_supported(device_ordinal)) {
    // a buffer that may be bound to a multicast object must honour that object's granularity too
    CUmulticastObjectProp mp = {};
    mp.numDevices = 2;
    mp.size = round_up(bytes, g);
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (d.cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > g) g = mg;
  }
  granularity_ = g;
  size_ = round_up(bytes, g);
  check(d.cuMemCreate(&local_handle_, size_, &prop, 0), "cuMemCreate");
  try {
    map_handle(local_handle_, &local_va_);
  } catch (...) {
    d.cuMemRelease(local_handle_);
    local_handle_ = 0;
    throw;
  }
}

void SymmetricBuffer::map_handle(CUmemGenericAllocationHandle h, CUdeviceptr* va) {
  const Driver& d = driver();
  check(d.cuMemAddressReserve(va, size_, granularity_, 0, 0), "cuMemAddressReserve");
  CUresult r = d.cuMemMap(*va, size_, 0, h, 0);
  if (r == CUDA_SUCCESS) {
    CUmemAccessDesc acc = {};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = ordinal_;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = d.cuMemSetAccess(*va, size_, &acc, 1);
    if (r != CUDA_SUCCESS) d.cuMemUnmap(*va, size_);
  }
  if (r != CUDA_SUCCESS) {
    d.cuMemAddressFree(*va, size_);
    *va = 0;
    check(r, "cuMemMap / cuMemSetAccess");
  }
}

int SymmetricBuffer::export_fd() {
  if (closed_) throw SpikeError("symmetric buffer is closed");
  int fd = -1;
  check(driver().cuMemExportToShareableHandle(&fd, local_handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
        "cuMemExportToShareableHandle");
  return fd;
}

void SymmetricBuffer::import_peer(int rank, int fd) {
  if (closed_) throw SpikeError("symmetric buffer is closed");
  if (rank < 0) throw SpikeError("negative peer rank");
  if (peer_ptr(rank) != 0) throw SpikeError("peer " + std::to_string(rank) + " was imported already");
  const Driver& d = driver();
  Peer p;
  p.rank = rank;
  check(d.cuMemImportFromShareableHandle(&p.handle, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                         CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
        "cuMemImportFromShareableHandle");
  try {
    map_handle(p.handle, &p.va);
  } catch (...) {
    d.cuMemRelease(p.handle);
    throw;
  }
  peers_.push_back(p);
}

uint64_t SymmetricBuffer::peer_ptr(int rank) const {
  for (const Peer& p : peers_)
    if (p.rank == rank) return static_cast<uint64_t>(p.va);
  return 0;
}

int SymmetricBuffer::multicast_create(int num_devices) {
  if (closed_) throw SpikeError("symmetric buffer is closed");
  const Driver& d = driver();
  if (!d.multicast_loaded) throw SpikeRuntimeError("this CUDA driver has no multicast API");
  if (mc_handle_) throw SpikeError("a multicast object exists already");
  CUmulticastObjectProp mp = {};
  mp.numDevices = static_cast<unsigned int>(num_devices);
  mp.size = size_;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  check(d.cuMulticastCreate(&mc_handle_, &mp), "cuMulticastCreate");
  int fd = -1;
  CUresult r = d.cuMemExportToShareableHandle(&fd, mc_handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    d.cuMemRelease(mc_handle_);
    mc_handle_ = 0;
    check(r, "cuMemExportToShareableHandle(multicast)");
  }
  return fd;
}

void SymmetricBuffer::multicast_import(int fd) {
  if (closed_) throw SpikeError("symmetric buffer is closed");
  if (mc_handle_) throw SpikeError("a multicast object exists already");
  check(driver().cuMemImportFromShareableHandle(&mc_handle_, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
        "cuMemImportFromShareableHandle(multicast)");
}

void SymmetricBuffer::multicast_add_device() {
  if (!mc_handle_) throw SpikeError("no multicast object");
  check(driver().cuMulticastAddDevice(mc_handle_, device_), "cuMulticastAddDevice");
}

void SymmetricBuffer::multicast_bind() {
  if (!mc_handle_) throw SpikeError("no multicast object");
  if (mc_bound_) return;
  const Driver& d = driver();
  check(d.cuMulticastBindMem(mc_handle_, 0, local_handle_, 0, size_, 0), "cuMulticastBindMem");
  mc_bound_ = true;
  map_handle(mc_handle_, &mc_va_);
}

void SymmetricBuffer::zero() {
  if (closed_) throw SpikeError("symmetric buffer is closed");
  const Driver& d = driver();
  check(d.cuMemsetD8_v2(local_va_, 0, size_), "cuMemsetD8");
  check(d.cuCtxSynchronize(), "cuCtxSynchronize");
}

void SymmetricBuffer::close() {
  if (closed_) return;
  closed_ = true;
  const Driver& d = driver();
  if (!d.loaded || !d.vmm_loaded) return;
  // order: the multicast view and binding first, then the peers' mappings, then the local memory
  if (mc_va_) {
    d.cuMemUnmap(mc_va_, size_);
    d.cuMemAddressFree(mc_va_, size_);
    mc_va_ = 0;
  }
  if (mc_handle_) {
    if (mc_bound_) d.cuMulticastUnbind(mc_handle_, device_, 0, size_);
    mc_bound_ = false;
    d.cuMemRelease(mc_handle_);
    mc_handle_ = 0;
  }
  for (Peer& p : peers_) {
    if (p.va) {
      d.cuMemUnmap(p.va, size_);
      d.cuMemAddressFree(p.va, size_);
    }
    if (p.handle) d.cuMemRelease(p.handle);
  }
  peers_.clear();
  if (local_va_) {
    d.cuMemUnmap(local_va_, size_);
    d.cuMemAddressFree(local_va_, size_);
    local_va_ = 0;
  }
  if (local_handle_) {
    d.cuMemRelease(local_handle_);
    local_handle_ = 0;
  }
}

SymmetricBuffer::~SymmetricBuffer() { close(); }

}  // namespace spike
