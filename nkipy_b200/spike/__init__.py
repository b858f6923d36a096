"""Device runtime: C++ core (`_spike`, csrc/runtime) with the Python conveniences of the
reference's `spike` package (spike/src/spike/__init__.py:1-30)."""

from .logger import get_logger
from .profiler_adapter import SpikeProfiler
from .spike_model import BenchmarkResult, SpikeModel
from .spike_singleton import configure, get_spike_singleton, reset, visible_device_count
from .spike_tensor import SpikeTensor


def __getattr__(name):
    # native types are resolved lazily so importing the package never needs the compiled module
    if name in ("SpikeError", "SpikeRuntimeError", "CudaError", "NrtError", "SystemTraceSession", "ModelTensorInfo",
                "NrtModel", "NrtTensor", "TensorMetadata", "Spike"):
        from .spike_singleton import _native

        return getattr(_native(), name)
    raise AttributeError(name)


__all__ = ["SpikeModel", "SpikeTensor", "SpikeProfiler", "configure", "reset", "get_spike_singleton", "NrtError",
           "SpikeError", "SystemTraceSession", "BenchmarkResult", "ModelTensorInfo", "NrtModel", "NrtTensor",
           "TensorMetadata", "get_logger", "visible_device_count"]
