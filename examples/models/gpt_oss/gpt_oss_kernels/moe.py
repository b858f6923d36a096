"""Routed feed-forward of gpt-oss for all tokens at once: top-k over the biased router logits, softmax over the
chosen k, expert projections with biases and the clamped activation (up + 1) * gate * sigmoid(alpha * gate)
(examples/models/gpt_oss/kernels/feedforward.py in the reference; the routing order differs from Qwen3's)."""
import numpy as np

from nkipy_b200.core import tensor_apis


def moe_ffn(x, router_weight, router_bias, gate_up_weight, gate_up_bias, down_weight, down_bias, top_k: int,
            limit: float, alpha: float):
    """x [B, T, H]; gate_up_weight [E, H, 2 I] (gate half first), gate_up_bias [E, 2 I]; down_weight [E, I, H],
    down_bias [E, H]."""
    B, T, H = x.shape
    N = B * T
    x2d = x.reshape(N, H)
    logits = (np.matmul(x2d, router_weight) + router_bias).astype(np.float32)
    top, idx = tensor_apis.topk(logits, top_k)
    w = tensor_apis.softmax(top)                                              # [N, K]
    gu = np.take(gate_up_weight, idx, axis=0)                                 # [N, K, H, 2 I]
    dn = np.take(down_weight, idx, axis=0)                                    # [N, K, I, H]
    bgu = np.take(gate_up_bias, idx, axis=0)                                  # [N, K, 2 I]
    bdn = np.take(down_bias, idx, axis=0)                                     # [N, K, H]
    xk = np.broadcast_to(x2d[:, None, None, :], (N, top_k, 1, H))
    h = np.matmul(xk, gu).reshape(N, top_k, -1) + bgu
    g, u = np.split(h, 2, axis=-1)
    g = np.minimum(g, np.float32(limit))
    u = np.clip(u, np.float32(-limit), np.float32(limit))
    a = (u + 1.0) * g * (1.0 / (1.0 + np.exp(-np.float32(alpha) * g)))
    y = np.matmul(a[:, :, None, :], dn).reshape(N, top_k, H) + bdn
    out = np.sum(y * w[:, :, None].astype(y.dtype), axis=1)
    return out.reshape(B, T, H)
