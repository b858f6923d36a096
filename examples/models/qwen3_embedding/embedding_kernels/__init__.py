"""Qwen3-Embedding as NumPy kernel functions for the tracing frontend: a padded batch goes through dense decoder
layers without a KV cache (causal attention with QK-norm), the hidden state of each sequence's last valid token is
picked and L2-normalised.  Counterpart of the reference's examples/models/qwen3_embedding/kernels/."""
from .encoder import encoder_layer, pool_and_normalize

__all__ = ["encoder_layer", "pool_and_normalize"]
