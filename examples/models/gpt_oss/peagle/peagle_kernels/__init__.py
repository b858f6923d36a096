"""The P-EAGLE drafter as NumPy kernel functions for the tracing frontend (the serving implementation is
`nkipy_b200/models/speculative.py`): fusion of token embeddings with the target's tapped hidden states, the fusion
layer whose attention reads both halves, a window of rows at a runtime position, and the draft-token head.
Counterpart of the reference's examples/models/gpt_oss/peagle/kernels/{drafter,drafter_layer}.py."""
from .drafter import draft_tokens, drafter_layer, fuse_inputs, fusion_layer, window_attention

__all__ = ["fuse_inputs", "window_attention", "fusion_layer", "drafter_layer", "draft_tokens"]
