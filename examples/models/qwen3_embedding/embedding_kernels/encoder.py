"""Encoder layer and pooling of the embedding model.

A layer is the dense decoder layer run once over the whole (right-padded) batch: RMSNorm, causal attention with
per-head QK-norm and RoPE, residual, RMSNorm, SwiGLU, residual.  There is no cache: keys and values are the
current tokens.  Padding tokens sit behind every valid token of their sequence, so the causal mask already hides
them from the tokens that are pooled (examples/models/qwen3_embedding/kernels/transformer_layer.py and
embedding_utils.py:6-30 in the reference: last-token pooling over the attention mask, then normalisation)."""
import numpy as np

from nkipy_b200.core import tensor_apis

from llama_kernels.feedforward import swiglu_ffn
from llama_kernels.rmsnorm import rmsnorm
from llama_kernels.rope import rope_tables, rotate_halves


def encoder_layer(x, qkv_weight, o_weight, q_norm, k_norm, gate_up_weight, down_weight, input_norm, post_norm,
                  n_heads: int, n_kv_heads: int, head_dim: int, rope_theta: float, norm_eps: float):
    """x [B, T, H] -> [B, T, H]."""
    B, T, _ = x.shape
    nq, nkv, D = n_heads, n_kv_heads, head_dim
    h = rmsnorm(x, input_norm, norm_eps)
    qkv = np.matmul(h, qkv_weight)
    q, k, v = np.split(qkv, [nq * D, (nq + nkv) * D], axis=-1)
    q, k, v = q.reshape(B, T, nq, D), k.reshape(B, T, nkv, D), v.reshape(B, T, nkv, D)
    q, k = rmsnorm(q, q_norm, norm_eps), rmsnorm(k, k_norm, norm_eps)
    cos, sin = rope_tables(D, T, rope_theta)
    cos_t, sin_t = cos[None, :, None, :], sin[None, :, None, :]
    q, k = rotate_halves(q, cos_t, sin_t), rotate_halves(k, cos_t, sin_t)
    rep = nq // nkv
    if rep > 1:
        k, v = np.repeat(k, rep, axis=2), np.repeat(v, rep, axis=2)
    scores = np.matmul(q.transpose(0, 2, 1, 3), k.transpose(0, 2, 3, 1)).astype(np.float32) * np.float32(1.0 / np.sqrt(D))
    pos = np.arange(T, dtype=np.int32)
    scores = np.where((pos[None, :] <= pos[:, None])[None, None], scores, np.float32(-1e30))
    p = tensor_apis.softmax(scores).astype(x.dtype)
    ctx = np.matmul(p, v.transpose(0, 2, 1, 3)).transpose(0, 2, 1, 3).reshape(B, T, nq * D)
    x = x + np.matmul(ctx, o_weight)
    return x + swiglu_ffn(rmsnorm(x, post_norm, norm_eps), gate_up_weight, down_weight)


def pool_and_normalize(x, last_index, final_norm, norm_eps: float):
    """x [B, T, H]; last_index int32 [B] (position of each sequence's last valid token).  Final norm of the pooled
    rows, then L2 normalisation; returns float32 [B, H]."""
    B, T, H = x.shape
    rows = np.arange(B, dtype=np.int32) * np.int32(T) + last_index
    pooled = np.take(x.reshape(B * T, H), rows, axis=0)
    e = rmsnorm(pooled, final_norm, norm_eps).astype(np.float32)
    return e / np.maximum(np.sqrt(np.sum(e * e, axis=-1, keepdims=True)), np.float32(1e-12))
