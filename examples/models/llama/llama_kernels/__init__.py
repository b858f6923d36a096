"""NumPy kernel functions of a Llama / Qwen3-style decoder, written against the tracing frontend: every function
here runs unchanged on NumPy arrays (CPU direct mode) and on traced tensors (compiled to CUDA)."""
from .attention import attention_block
from .feedforward import swiglu_ffn
from .rmsnorm import rmsnorm
from .rope import rope_tables, rotate_halves
from .sampling import greedy_token
from .transformer_layer import decode_layer, prefill_layer

__all__ = ["attention_block", "swiglu_ffn", "rmsnorm", "rope_tables", "rotate_halves", "greedy_token", "decode_layer",
           "prefill_layer"]
