// A loaded kernel: cubin + launch plan.
//
// Counterpart of the reference's NrtModel (spike/src/model.cpp:10-150: read NEFF, load it on
// a core — optionally with rank / world size for collectives —, execute with named input and
// output tensor sets, optional profile capture, tensor info query, unload).  Here the unit
// is a cubin produced by nvcc from generated CUDA C++ plus a JSON sidecar listing buffers
// (inputs, outputs, temporaries, constants), the ordered kernel launches with their
// arguments (buffer pointers, scalars, TMA tensor maps, GEMM argument blocks) and the
// input/output alias pairs.
#pragma once
#include <cuda.h>

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "json.h"
#include "runtime.h"
#include "trace.h"

namespace spike {

struct TensorMetadata {
  size_t size = 0;
  std::string dtype;
  std::vector<long long> shape;
};

struct ModelTensorInfo {
  std::map<std::string, TensorMetadata> inputs;
  std::map<std::string, TensorMetadata> outputs;
  std::vector<std::string> input_order;
  std::vector<std::string> output_order;
  std::map<std::string, std::string> aliases;   // output name -> input name sharing its buffer
};

class LoadedModule {
 public:
  LoadedModule(const CudaRuntime& rt, const std::string& path, int core_id, bool cc_enabled, int rank_id,
               int world_size);
  ~LoadedModule();
  LoadedModule(const LoadedModule&) = delete;
  LoadedModule& operator=(const LoadedModule&) = delete;

  // Runs the plan on the runtime's stream and waits for it.  With save_trace the per-launch
  // device times are written to `trace_path` as JSON.
  void execute(const TensorSet& inputs, const TensorSet& outputs, const std::string& trace_path, bool save_trace);
  ModelTensorInfo tensor_info() const { return info_; }
  void unload();
  bool unloaded() const { return module_ == nullptr; }

  const std::string& path() const { return path_; }
  const std::string& name() const { return name_; }
  int core_id() const { return core_id_; }
  int rank_id() const { return rank_id_; }
  int world_size() const { return world_size_; }
  bool is_collective() const { return cc_enabled_; }
  size_t num_launches() const { return launches_.size(); }

  // Collectives inside the module (plan section "collective"): the symmetric workspace of every rank of the
  // group, in rank order (peer_ws[rank] is this process's own mapping), each `workspace_bytes()` long and zeroed.
  // Modules traced for one rank get a private workspace automatically.  Called once, before the first execute.
  void set_collective_workspace(const std::vector<unsigned long long>& peer_ws);
  bool has_collectives() const { return cc_world_ > 0; }
  int collective_world() const { return cc_world_; }
  size_t workspace_bytes() const { return cc_workspace_bytes_; }

 private:
  struct Buf {
    size_t nbytes = 0;
    std::string kind, name;
    int alias_of = -1;
    CUdeviceptr owned = 0;     // temp / const storage owned by the module
  };
  struct Arg {
    enum Kind { Buffer, I32, I64, F32, TensorMap, GemmArgs, CcTable } kind = Buffer;
    int buffer = -1;
    long long offset = 0;
    long long ival = 0;
    double fval = 0;
    std::vector<unsigned long long> dims, strides;
    std::vector<unsigned> box;
    Json gemm;
  };
  struct LaunchRec {
    std::string kernel, loc;
    CUfunction fn = nullptr;
    unsigned grid[3] = {1, 1, 1}, block[3] = {1, 1, 1};
    unsigned smem = 0;
    std::vector<Arg> args;
  };

  const CudaRuntime& rt_;
  std::string path_, name_;
  int core_id_, rank_id_, world_size_;
  bool cc_enabled_;
  CUmodule module_ = nullptr;
  std::vector<Buf> bufs_;
  std::vector<LaunchRec> launches_;
  ModelTensorInfo info_;
  std::map<std::string, int> input_buf_, output_buf_;
  std::shared_ptr<std::atomic<bool>> runtime_closed_;
  // collectives: device copy of the table the generated kernels read, its counters, a private workspace
  int cc_world_ = 0;
  size_t cc_workspace_bytes_ = 0, cc_half_bytes_ = 0;
  CUdeviceptr cc_table_ = 0, cc_counters_ = 0, cc_private_ws_ = 0;
};

}  // namespace spike
