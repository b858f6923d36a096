"""Tracing frontend: kernels are plain NumPy functions that run directly on arrays (CPU
direct mode) or are traced into the tensor IR of `nkipy_b200.core.ir`."""
