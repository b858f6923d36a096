"""Attention block of gpt-oss: fused QKV with bias, RoPE from host-built (YaRN) tables, a dense cache written in
place, a causal mask that may be cut to a sliding window, and a learnt sink logit per head that takes part in the
softmax but contributes no value (examples/models/gpt_oss/kernels/attention.py:116-148 in the reference)."""
import numpy as np

from nkipy_b200.core import tensor_apis

from llama_kernels.rope import rotate_halves


def attention_block(x, qkv_weight, qkv_bias, o_weight, o_bias, sinks, cos, sin, cache_k, cache_v, start_pos, *,
                    n_heads: int, n_kv_heads: int, head_dim: int, window: int):
    """x [B, T, H]; cos / sin [S_max, D / 2]; sinks [nq] float32; caches [B, S_max, nkv, D]; start_pos None = prefill,
    else int32 [1]; window 0 = full attention.  Returns the block output [B, T, H] before the residual add."""
    B, T, _ = x.shape
    S = cache_k.shape[1]
    nq, nkv, D = n_heads, n_kv_heads, head_dim
    qkv = np.matmul(x, qkv_weight) + qkv_bias
    q, k, v = np.split(qkv, [nq * D, (nq + nkv) * D], axis=-1)
    q, k, v = q.reshape(B, T, nq, D), k.reshape(B, T, nkv, D), v.reshape(B, T, nkv, D)
    if start_pos is None:
        cos_t, sin_t = cos[:T][None, :, None, :], sin[:T][None, :, None, :]
    else:
        cos_t, sin_t = cos[start_pos][None, :, None, :], sin[start_pos][None, :, None, :]
    q, k = rotate_halves(q, cos_t, sin_t), rotate_halves(k, cos_t, sin_t)
    if start_pos is None:
        cache_k[:, :T] = k
        cache_v[:, :T] = v
    else:
        cache_k[:, start_pos] = k
        cache_v[:, start_pos] = v
    rep = nq // nkv
    keys = np.repeat(cache_k, rep, axis=2) if rep > 1 else cache_k
    vals = np.repeat(cache_v, rep, axis=2) if rep > 1 else cache_v
    qh = q.transpose(0, 2, 1, 3)                                             # [B, nq, T, D]
    kh = keys.transpose(0, 2, 3, 1)                                          # [B, nq, D, S]
    vh = vals.transpose(0, 2, 1, 3)                                          # [B, nq, S, D]
    scores = np.matmul(qh, kh).astype(np.float32) * np.float32(1.0 / np.sqrt(D))
    key_pos = np.arange(S, dtype=np.int32)
    if start_pos is None:
        q_pos = np.arange(T, dtype=np.int32)[:, None]                          # trace-time constants
        visible = key_pos[None, :] <= q_pos
        if window > 0:
            visible = visible & (key_pos[None, :] > q_pos - window)
    else:
        kp = tensor_apis.constant(key_pos)[None, :]
        visible = kp <= start_pos[:, None]
        if window > 0:
            visible = visible & (kp > start_pos[:, None] - np.int32(window))
    scores = np.where(visible[None, None], scores, np.float32(-1e30))
    # softmax over the keys and one more logit per head, the sink, which only enlarges the denominator
    sink = sinks.astype(np.float32)[None, :, None, None]
    m = np.maximum(np.max(scores, axis=-1, keepdims=True), sink)
    e = np.exp(scores - m)
    p = (e / (np.sum(e, axis=-1, keepdims=True) + np.exp(sink - m))).astype(x.dtype)
    ctx = np.matmul(p, vh).transpose(0, 2, 1, 3).reshape(B, T, nq * D)
    return np.matmul(ctx, o_weight) + o_bias
