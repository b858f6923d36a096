"""Back-compat re-exports of ops that have no NumPy spelling
(nkipy/src/nkipy/core/tensor_apis.py:5-25 in the reference)."""

from .ops import (constant, conv2d, conv3d, erf, full, gelu, ones, rms_norm, rsqrt, sigmoid, silu, softmax, topk,
                  zeros)

__all__ = ["constant", "topk", "rms_norm", "softmax", "conv2d", "conv3d", "zeros", "full", "ones", "erf", "rsqrt",
           "sigmoid", "silu", "gelu"]
