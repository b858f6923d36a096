"""RMSNorm over the last axis with fp32 statistics (same arithmetic as the reference's
examples/models/qwen3/kernels/rmsnorm.py:4-21: mean of squares, eps inside the root, weight, cast back)."""
import numpy as np


def rmsnorm(x, weight, eps: float):
    xf = x.astype(np.float32)
    inv = 1.0 / np.sqrt(np.mean(xf * xf, axis=-1, keepdims=True) + np.float32(eps))
    return (xf * inv * weight.astype(np.float32)).astype(x.dtype)
