// Runtime facade: one live instance per process owns the CUDA context, creates tensors and
// models and executes them.  Same surface as the reference's spike::Spike
// (spike/src/include/spike.h:29-91, spike/src/spike.cpp:1-187): load_model,
// allocate_tensor, slice_from_tensor, free_tensor, tensor_write / tensor_read, execute
// (rejects freed tensors), get_tensor_info, close.
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "module.h"
#include "runtime.h"
#include "trace.h"

namespace spike {

class Spike {
 public:
  explicit Spike(int verbose_level = 0, int device_ordinal = -1);
  ~Spike();
  Spike(const Spike&) = delete;
  Spike& operator=(const Spike&) = delete;

  static int get_visible_neuron_core_count();   // number of CUDA devices this process can see
  int device_ordinal() const;
  std::string device_name() const;
  int sm_count() const;
  size_t total_memory() const;

  std::shared_ptr<LoadedModule> load_model(const std::string& path, int core_id, bool cc_enabled, int rank_id,
                                           int world_size);
  void unload_model(const std::shared_ptr<LoadedModule>& model);
  std::shared_ptr<DeviceBuffer> allocate_tensor(size_t size, int core_id, const std::string& name);
  std::shared_ptr<DeviceBuffer> slice_from_tensor(const std::shared_ptr<DeviceBuffer>& src, size_t offset, size_t size,
                                                  const std::string& name);
  void free_tensor(const std::shared_ptr<DeviceBuffer>& t);
  void tensor_write(const std::shared_ptr<DeviceBuffer>& t, const void* data, size_t size, size_t offset);
  void tensor_read(const std::shared_ptr<DeviceBuffer>& t, void* data, size_t size, size_t offset);
  void execute(const std::shared_ptr<LoadedModule>& model,
               const std::vector<std::pair<std::string, std::shared_ptr<DeviceBuffer>>>& inputs,
               const std::vector<std::pair<std::string, std::shared_ptr<DeviceBuffer>>>& outputs,
               const std::string& trace_path, bool save_trace);
  ModelTensorInfo get_tensor_info(const std::shared_ptr<LoadedModule>& model);
  int read_status(bool reset);
  void close();
  bool is_closed() const { return closed_; }

 private:
  void require_open(const char* what) const;
  std::unique_ptr<CudaRuntime> rt_;
  bool closed_ = false;
  int verbose_;
};

}  // namespace spike
