"""gpt-oss as NumPy kernel functions for the tracing frontend: attention with biases, a sliding window on
alternating layers and per-head sink logits; routing by top-k over the logits and a softmax over the chosen ones;
expert feed-forward with biases and the clamped activation.  Counterpart of the reference's
examples/models/gpt_oss/kernels/."""
from .attention import attention_block
from .moe import moe_ffn
from .transformer_layer import decode_layer, prefill_layer
from .verify import accept, verify_tokens

__all__ = ["attention_block", "moe_ffn", "prefill_layer", "decode_layer", "verify_tokens", "accept"]
