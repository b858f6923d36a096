"""Final norm, LM head and greedy choice of the next token for the last position of every sequence
(examples/models/qwen3/kernels/sampling.py in the reference)."""
import numpy as np

from .rmsnorm import rmsnorm


def greedy_token(x, final_norm, lm_head, norm_eps: float):
    """x [B, T, H]; lm_head [H, V].  Returns int32 [B]."""
    last = x[:, -1, :]
    logits = np.matmul(rmsnorm(last, final_norm, norm_eps), lm_head).astype(np.float32)
    return np.argmax(logits, axis=-1).astype(np.int32)
