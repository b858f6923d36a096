// Error hierarchy of the device runtime, surfaced to Python as exceptions.
// (Reference: spike/src/include/error.h:12-43 has SpikeRuntimeError > SpikeError and
// NrtError carrying the vendor status code; here the vendor code is a CUresult.)
#pragma once
#include <stdexcept>
#include <string>

namespace spike {

class SpikeRuntimeError : public std::runtime_error {
 public:
  explicit SpikeRuntimeError(const std::string& msg) : std::runtime_error(msg) {}
};

// Misuse of the runtime API: freed tensors, closed runtime, bad names or sizes.
class SpikeError : public SpikeRuntimeError {
 public:
  explicit SpikeError(const std::string& msg) : SpikeRuntimeError(msg) {}
};

// A CUDA driver call failed.
class CudaError : public SpikeRuntimeError {
 public:
  CudaError(int code, const std::string& msg) : SpikeRuntimeError(msg), code_(code) {}
  int code() const { return code_; }

 private:
  int code_;
};

}  // namespace spike
