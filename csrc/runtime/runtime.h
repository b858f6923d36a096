// Core RAII objects of the device runtime: the per-process CUDA context holder,
// device buffers (owning allocations and non-owning slices), and named tensor sets.
//
// Counterparts in the reference: NrtRuntime (spike/src/nrt_wrapper.cpp:49-76),
// NrtTensor with slice views and the "runtime closed" token that turns late
// destructors into no-ops (spike/src/tensor.cpp:9-125), NrtTensorSet
// (spike/src/tensor_set.cpp:5-40).  One process drives one GPU; `core_id` is kept in
// the API for parity and must name the device chosen at initialisation.
#pragma once
#include <cuda.h>

#include <atomic>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "driver.h"
#include "error.h"

namespace spike {

class CudaRuntime {
 public:
  explicit CudaRuntime(int device_ordinal);
  ~CudaRuntime();
  CudaRuntime(const CudaRuntime&) = delete;
  CudaRuntime& operator=(const CudaRuntime&) = delete;

  static int visible_device_count();
  int device_ordinal() const { return ordinal_; }
  CUdevice device() const { return device_; }
  CUcontext context() const { return ctx_; }
  CUstream stream() const { return stream_; }
  std::string device_name() const;
  size_t total_memory() const;
  int sm_count() const;
  void make_current() const;
  void synchronize() const;
  // shared flag flipped at close(): buffers and modules outliving the runtime skip their frees
  std::shared_ptr<std::atomic<bool>> closed_token() const { return closed_; }
  int* status_word() const { return reinterpret_cast<int*>(status_); }
  int read_status(bool reset) const;
  void close();

 private:
  int ordinal_;
  CUdevice device_ = 0;
  CUcontext ctx_ = nullptr;
  CUstream stream_ = nullptr;
  CUdeviceptr status_ = 0;
  std::shared_ptr<std::atomic<bool>> closed_;
};

class DeviceBuffer {
 public:
  // owning allocation
  DeviceBuffer(const CudaRuntime& rt, size_t size, std::string name, int core_id);
  // non-owning view of [offset, offset + size) of `parent`
  DeviceBuffer(const std::shared_ptr<DeviceBuffer>& parent, size_t offset, size_t size, std::string name);
  ~DeviceBuffer();
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;

  void write(const void* src, size_t size, size_t offset = 0);
  void read(void* dst, size_t size, size_t offset = 0) const;
  void free();
  bool is_freed() const;

  size_t size() const { return size_; }
  const std::string& name() const { return name_; }
  int core_id() const { return core_id_; }
  uint64_t va() const { return static_cast<uint64_t>(ptr_); }
  CUdeviceptr ptr() const { return ptr_; }

 private:
  void require_live(const char* what) const;
  CUdeviceptr ptr_ = 0;
  size_t size_ = 0;
  std::string name_;
  int core_id_ = 0;
  bool owner_ = true;
  bool freed_ = false;
  std::shared_ptr<DeviceBuffer> parent_;
  std::shared_ptr<std::atomic<bool>> runtime_closed_;
};

// name -> buffer, as passed to LoadedModule::execute
class TensorSet {
 public:
  void add(const std::string& name, std::shared_ptr<DeviceBuffer> buf);
  std::shared_ptr<DeviceBuffer> get(const std::string& name) const;
  bool has(const std::string& name) const { return map_.count(name) != 0; }
  size_t size() const { return map_.size(); }
  const std::map<std::string, std::shared_ptr<DeviceBuffer>>& items() const { return map_; }

 private:
  std::map<std::string, std::shared_ptr<DeviceBuffer>> map_;
};

}  // namespace spike
