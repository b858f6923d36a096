"""Routed feed-forward of Qwen3-MoE as one kernel function for all tokens at once.

The reference walks over batch, tokens and selected experts in Python and indexes the expert weights with a traced
scalar (examples/models/qwen3/kernels/transformer_layer.py:74-106 there), which unrolls B x T x top_k expert
feed-forwards into the graph.  Here the routing is a softmax + top-k over all tokens, the selected experts' weights
are gathered with `np.take` and the two projections are batched matrix products over (token, slot), so the graph
has a fixed size whatever the batch is."""
import numpy as np

from nkipy_b200.core import tensor_apis


def route(x2d, router_weight, top_k: int):
    """x2d [N, H] -> (weights [N, top_k] summing to one, expert ids [N, top_k]): softmax over all experts, then the
    top-k probabilities renormalised (Qwen3's order; gpt-oss takes the top-k logits first)."""
    probs = tensor_apis.softmax(np.matmul(x2d, router_weight).astype(np.float32))
    w, idx = tensor_apis.topk(probs, top_k)
    return w / np.sum(w, axis=-1, keepdims=True), idx


def moe_ffn(x, router_weight, gate_up_weight, down_weight, top_k: int):
    """x [B, T, H]; router_weight [H, E]; gate_up_weight [E, H, 2 I]; down_weight [E, I, H] -> [B, T, H]."""
    B, T, H = x.shape
    N = B * T
    x2d = x.reshape(N, H)
    w, idx = route(x2d, router_weight, top_k)
    gu = np.take(gate_up_weight, idx, axis=0)                       # [N, K, H, 2 I]
    dn = np.take(down_weight, idx, axis=0)                          # [N, K, I, H]
    xk = np.broadcast_to(x2d[:, None, None, :], (N, top_k, 1, H))
    g, u = np.split(np.matmul(xk, gu), 2, axis=-1)                  # [N, K, 1, I] each
    a = g * (1.0 / (1.0 + np.exp(-g))) * u
    y = np.matmul(a, dn).reshape(N, top_k, H)
    out = np.sum(y * w[:, :, None].astype(y.dtype), axis=1)
    return out.reshape(B, T, H)
