"""Qwen3-MoE as NumPy kernel functions for the tracing frontend: the attention block, the norms, RoPE and the sampler
are the ones of the Llama example (`examples/models/llama/llama_kernels`, attention with per-head QK-norm); this
package adds the routed feed-forward and the layer that uses it.  Counterpart of the reference's
examples/models/qwen3/kernels/."""
from .moe import moe_ffn, route
from .transformer_layer import decode_layer, prefill_layer

__all__ = ["moe_ffn", "route", "prefill_layer", "decode_layer"]
