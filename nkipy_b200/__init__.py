"""nkipy_b200: a Blackwell-native NumPy-style kernel framework.

Sub-packages: ``core`` (tracing frontend + IR), ``compiler`` (IR -> CUDA C++),
``runtime`` (JIT / device kernels / device tensors), ``ops`` (hand-written
sm_100a kernels), ``models`` (Llama-style dense, Qwen3-style MoE, gpt-oss-style,
embedding, linear attention), ``parallel`` (tensor / expert / sequence
parallelism and fused compute+collective kernels), ``distributed`` (collective
ops), ``utils``.
"""

__version__ = "0.1.0"

from .core.knob import knob  # noqa: E402,F401
