"""Python runtime API (nkipy/src/nkipy/runtime/__init__.py:15-23 in the reference)."""

from .baremetal_executor import BaremetalExecutor, CompiledKernel
from .decorators import baremetal_jit
from .device_kernel import DeviceKernel
from .device_tensor import DeviceTensor
from .execute import baremetal_run_traced_kernel
from .segmented import SegmentedKernel
from .utils import is_device_compatible, is_neuron_compatible

__all__ = ["baremetal_jit", "baremetal_run_traced_kernel", "BaremetalExecutor", "CompiledKernel", "DeviceKernel",
           "DeviceTensor", "SegmentedKernel", "is_neuron_compatible", "is_device_compatible"]
