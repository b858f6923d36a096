"""RMSNorm over the last axis with fp32 statistics (same arithmetic as the reference's
examples/models/qwen3/kernels/rmsnorm.py:4-21: mean of squares, eps inside the root, weight, cast back).
`tensor_apis.rms_norm` is NumPy in direct mode and one row kernel when the function is compiled."""
from nkipy_b200.core import tensor_apis


def rmsnorm(x, weight, eps: float):
    return tensor_apis.rms_norm(x, weight, eps)
