#include "runtime.h"

#include <utility>

namespace spike {

int CudaRuntime::visible_device_count() {
  const Driver& d = driver();
  if (!d.loaded) return 0;
  if (d.cuInit(0) != CUDA_SUCCESS) return 0;
  int n = 0;
  if (d.cuDeviceGetCount(&n) != CUDA_SUCCESS) return 0;
  return n;
}

CudaRuntime::CudaRuntime(int device_ordinal) : ordinal_(device_ordinal), closed_(std::make_shared<std::atomic<bool>>(false)) {
  const Driver& d = driver();
  if (!d.loaded) throw SpikeRuntimeError("CUDA driver library could not be loaded: " + d.load_error);
  check(d.cuInit(0), "cuInit");
  int n = 0;
  check(d.cuDeviceGetCount(&n), "cuDeviceGetCount");
  if (device_ordinal < 0 || device_ordinal >= n)
    throw SpikeError("device ordinal " + std::to_string(device_ordinal) + " out of range (" + std::to_string(n) +
                     " visible)");
  check(d.cuDeviceGet(&device_, device_ordinal), "cuDeviceGet");
  check(d.cuDevicePrimaryCtxRetain(&ctx_, device_), "cuDevicePrimaryCtxRetain");
  check(d.cuCtxSetCurrent(ctx_), "cuCtxSetCurrent");
  check(d.cuStreamCreate(&stream_, CU_STREAM_NON_BLOCKING), "cuStreamCreate");
  check(d.cuMemAlloc_v2(&status_, 64), "cuMemAlloc(status)");
  check(d.cuMemsetD8_v2(status_, 0, 64), "cuMemsetD8(status)");
}

void CudaRuntime::close() {
  if (closed_->exchange(true)) return;
  const Driver& d = driver();
  if (ctx_) {
    d.cuCtxSetCurrent(ctx_);
    d.cuCtxSynchronize();
    if (status_) d.cuMemFree_v2(status_);
    if (stream_) d.cuStreamDestroy_v2(stream_);
    d.cuDevicePrimaryCtxRelease_v2(device_);
  }
  ctx_ = nullptr;
  stream_ = nullptr;
  status_ = 0;
}

CudaRuntime::~CudaRuntime() { close(); }

void CudaRuntime::make_current() const {
  if (closed_->load()) throw SpikeError("runtime is closed");
  check(driver().cuCtxSetCurrent(ctx_), "cuCtxSetCurrent");
}

void CudaRuntime::synchronize() const {
  make_current();
  check(driver().cuStreamSynchronize(stream_), "cuStreamSynchronize");
}

std::string CudaRuntime::device_name() const {
  char buf[256] = {0};
  check(driver().cuDeviceGetName(buf, 255, device_), "cuDeviceGetName");
  return buf;
}

size_t CudaRuntime::total_memory() const {
  size_t n = 0;
  check(driver().cuDeviceTotalMem_v2(&n, device_), "cuDeviceTotalMem");
  return n;
}

int CudaRuntime::sm_count() const {
  int n = 0;
  check(driver().cuDeviceGetAttribute(&n, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, device_), "cuDeviceGetAttribute");
  return n;
}

int CudaRuntime::read_status(bool reset) const {
  make_current();
  int v = 0;
  check(driver().cuMemcpyDtoH_v2(&v, status_, sizeof(int)), "cuMemcpyDtoH(status)");
  if (reset && v) check(driver().cuMemsetD8_v2(status_, 0, sizeof(int)), "cuMemsetD8(status)");
  return v;
}

// ---------------------------------------------------------------------------- DeviceBuffer
DeviceBuffer::DeviceBuffer(const CudaRuntime& rt, size_t size, std::string name, int core_id)
    : size_(size), name_(std::move(name)), core_id_(core_id), owner_(true), runtime_closed_(rt.closed_token()) {
  rt.make_current();
  check(driver().cuMemAlloc_v2(&ptr_, size ? size : 1), "cuMemAlloc");
}

DeviceBuffer::DeviceBuffer(const std::shared_ptr<DeviceBuffer>& parent, size_t offset, size_t size, std::string name)
    : size_(size), name_(std::move(name)), core_id_(parent->core_id_), owner_(false), parent_(parent),
      runtime_closed_(parent->runtime_closed_) {
  if (parent->is_freed()) throw SpikeError("cannot slice freed tensor '" + parent->name() + "'");
  if (offset > parent->size() || size > parent->size() - offset)
    throw SpikeError("slice [" + std::to_string(offset) + ", +" + std::to_string(size) + ") exceeds tensor '" +
                     parent->name() + "' of " + std::to_string(parent->size()) + " bytes");
  ptr_ = parent->ptr_ + offset;
}

bool DeviceBuffer::is_freed() const {
  if (freed_ || runtime_closed_->load()) return true;
  return parent_ ? parent_->is_freed() : false;
}

void DeviceBuffer::free() {
  if (freed_) return;
  freed_ = true;
  if (owner_ && !runtime_closed_->load() && ptr_) driver().cuMemFree_v2(ptr_);
  ptr_ = 0;
}

DeviceBuffer::~DeviceBuffer() { free(); }

void DeviceBuffer::require_live(const char* what) const {
  if (is_freed()) throw SpikeError(std::string(what) + ": tensor '" + name_ + "' was freed or the runtime is closed");
}

void DeviceBuffer::write(const void* src, size_t size, size_t offset) {
  require_live("write");
  if (offset > size_ || size > size_ - offset)
    throw SpikeError("write of " + std::to_string(size) + " bytes at offset " + std::to_string(offset) +
                     " exceeds tensor '" + name_ + "' of " + std::to_string(size_) + " bytes");
  if (size) check(driver().cuMemcpyHtoD_v2(ptr_ + offset, src, size), "cuMemcpyHtoD");
}

void DeviceBuffer::read(void* dst, size_t size, size_t offset) const {
  require_live("read");
  if (offset > size_ || size > size_ - offset)
    throw SpikeError("read of " + std::to_string(size) + " bytes at offset " + std::to_string(offset) +
                     " exceeds tensor '" + name_ + "' of " + std::to_string(size_) + " bytes");
  if (size) check(driver().cuMemcpyDtoH_v2(dst, ptr_ + offset, size), "cuMemcpyDtoH");
}

// ---------------------------------------------------------------------------- TensorSet
void TensorSet::add(const std::string& name, std::shared_ptr<DeviceBuffer> buf) {
  if (!buf) throw SpikeError("tensor set: null tensor for '" + name + "'");
  if (buf->is_freed()) throw SpikeError("tensor set: tensor '" + name + "' was freed");
  map_[name] = std::move(buf);
}

std::shared_ptr<DeviceBuffer> TensorSet::get(const std::string& name) const {
  auto it = map_.find(name);
  if (it == map_.end()) throw SpikeError("tensor set: no tensor named '" + name + "'");
  return it->second;
}

}  // namespace spike
