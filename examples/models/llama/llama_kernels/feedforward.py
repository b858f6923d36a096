"""SwiGLU feed-forward block: silu(x Wg) * (x Wu), then Wd
(examples/models/qwen3/kernels/feedforward.py:4-18 in the reference)."""
import numpy as np


def swiglu_ffn(x, gate_up_weight, down_weight):
    """x [..., H]; gate_up_weight [H, 2 I] (gate columns first); down_weight [I, H]."""
    gu = np.matmul(x, gate_up_weight)
    inter = gate_up_weight.shape[1] // 2
    g, u = gu[..., :inter].astype(np.float32), gu[..., inter:].astype(np.float32)
    act = (g / (1.0 + np.exp(-g)) * u).astype(x.dtype)
    return np.matmul(act, down_weight)
