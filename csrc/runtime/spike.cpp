#include "spike.h"

#include <cstdlib>
#include <mutex>

namespace spike {

static std::mutex g_alive_mu;
static bool g_alive = false;

static int pick_device(int requested) {
  if (requested >= 0) return requested;
  // one process drives one GPU: LOCAL_RANK picks it under torchrun, default device 0
  if (const char* lr = std::getenv("LOCAL_RANK")) {
    int n = CudaRuntime::visible_device_count();
    int r = std::atoi(lr);
    if (n > 0) return r % n;
  }
  return 0;
}

Spike::Spike(int verbose_level, int device_ordinal) : verbose_(verbose_level) {
  std::lock_guard<std::mutex> lock(g_alive_mu);
  if (g_alive) throw SpikeError("only one Spike runtime instance may be alive in a process");
  rt_ = std::make_unique<CudaRuntime>(pick_device(device_ordinal));
  g_alive = true;
}

Spike::~Spike() { close(); }

void Spike::close() {
  if (closed_) return;
  closed_ = true;
  if (rt_) rt_->close();
  std::lock_guard<std::mutex> lock(g_alive_mu);
  g_alive = false;
}

void Spike::require_open(const char* what) const {
  if (closed_) throw SpikeError(std::string(what) + ": runtime is closed");
}

int Spike::get_visible_neuron_core_count() { return CudaRuntime::visible_device_count(); }
int Spike::device_ordinal() const { return rt_->device_ordinal(); }
std::string Spike::device_name() const { require_open("device_name"); return rt_->device_name(); }
int Spike::sm_count() const { require_open("sm_count"); return rt_->sm_count(); }
size_t Spike::total_memory() const { require_open("total_memory"); return rt_->total_memory(); }

std::shared_ptr<LoadedModule> Spike::load_model(const std::string& path, int core_id, bool cc_enabled, int rank_id,
                                                int world_size) {
  require_open("load_model");
  return std::make_shared<LoadedModule>(*rt_, path, core_id, cc_enabled, rank_id, world_size);
}

void Spike::unload_model(const std::shared_ptr<LoadedModule>& model) {
  require_open("unload_model");
  model->unload();
}

std::shared_ptr<DeviceBuffer> Spike::allocate_tensor(size_t size, int core_id, const std::string& name) {
  require_open("allocate_tensor");
  if (core_id != 0 && core_id != rt_->device_ordinal())
    throw SpikeError("core_id " + std::to_string(core_id) + " is not the device this process drives");
  return std::make_shared<DeviceBuffer>(*rt_, size, name, core_id);
}

std::shared_ptr<DeviceBuffer> Spike::slice_from_tensor(const std::shared_ptr<DeviceBuffer>& src, size_t offset,
                                                       size_t size, const std::string& name) {
  require_open("slice_from_tensor");
  return std::make_shared<DeviceBuffer>(src, offset, size, name);
}

void Spike::free_tensor(const std::shared_ptr<DeviceBuffer>& t) {
  require_open("free_tensor");
  rt_->make_current();
  t->free();
}

void Spike::tensor_write(const std::shared_ptr<DeviceBuffer>& t, const void* data, size_t size, size_t offset) {
  require_open("tensor_write");
  rt_->make_current();
  t->write(data, size, offset);
}

void Spike::tensor_read(const std::shared_ptr<DeviceBuffer>& t, void* data, size_t size, size_t offset) {
  require_open("tensor_read");
  rt_->make_current();
  t->read(data, size, offset);
}

void Spike::execute(const std::shared_ptr<LoadedModule>& model,
                    const std::vector<std::pair<std::string, std::shared_ptr<DeviceBuffer>>>& inputs,
                    const std::vector<std::pair<std::string, std::shared_ptr<DeviceBuffer>>>& outputs,
                    const std::string& trace_path, bool save_trace) {
  require_open("execute");
  TensorSet in, out;
  for (auto& kv : inputs) in.add(kv.first, kv.second);
  for (auto& kv : outputs) out.add(kv.first, kv.second);
  model->execute(in, out, trace_path, save_trace);
}

ModelTensorInfo Spike::get_tensor_info(const std::shared_ptr<LoadedModule>& model) {
  require_open("get_tensor_info");
  return model->tensor_info();
}

int Spike::read_status(bool reset) {
  require_open("read_status");
  return rt_->read_status(reset);
}

}  // namespace spike
