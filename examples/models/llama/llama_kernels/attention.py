"""Grouped-query attention block with a dense KV cache that the kernel updates in place.

prefill: the whole prompt at once (positions 0 .. T-1, causal mask built at trace time);
decode:  one token per sequence at the runtime position `start_pos` (int32 [1]); the mask lets a query see
cache positions <= start_pos.  The cache arguments are written through (`cache[...] = ...`), which the
runtime maps onto the caller's device tensors (the reference's kernels do the same:
examples/models/qwen3/kernels/attention.py:100-106)."""
import numpy as np

from nkipy_b200.core import tensor_apis

from .rmsnorm import rmsnorm
from .rope import rope_tables, rotate_halves


def attention_block(x, qkv_weight, o_weight, cache_k, cache_v, start_pos, *, n_heads: int, n_kv_heads: int,
                    head_dim: int, rope_theta: float, q_norm=None, k_norm=None, norm_eps: float = 1e-6):
    """x [B, T, H]; qkv_weight [H, (nq + 2 nkv) D]; o_weight [nq D, H]; caches [B, S_max, nkv, D].
    start_pos None = prefill.  Returns the block output [B, T, H] (before the residual add)."""
    B, T, _ = x.shape
    S = cache_k.shape[1]
    nq, nkv, D = n_heads, n_kv_heads, head_dim
    qkv = np.matmul(x, qkv_weight)
    q, k, v = np.split(qkv, [nq * D, (nq + nkv) * D], axis=-1)
    q, k, v = q.reshape(B, T, nq, D), k.reshape(B, T, nkv, D), v.reshape(B, T, nkv, D)
    if q_norm is not None:
        q, k = rmsnorm(q, q_norm, norm_eps), rmsnorm(k, k_norm, norm_eps)
    cos, sin = rope_tables(D, S, rope_theta)
    if start_pos is None:
        cos_t, sin_t = cos[:T][None, :, None, :], sin[:T][None, :, None, :]
    else:
        cos_t = tensor_apis.constant(cos)[start_pos][None, :, None, :]        # [1, 1, 1, D / 2]
        sin_t = tensor_apis.constant(sin)[start_pos][None, :, None, :]
    q, k = rotate_halves(q, cos_t, sin_t), rotate_halves(k, cos_t, sin_t)
    if start_pos is None:
        cache_k[:, :T] = k
        cache_v[:, :T] = v
    else:
        cache_k[:, start_pos] = k
        cache_v[:, start_pos] = v
    rep = nq // nkv
    keys = np.repeat(cache_k, rep, axis=2) if rep > 1 else cache_k           # [B, S, nq, D]
    vals = np.repeat(cache_v, rep, axis=2) if rep > 1 else cache_v
    qh = q.transpose(0, 2, 1, 3)                                             # [B, nq, T, D]
    kh = keys.transpose(0, 2, 3, 1)                                          # [B, nq, D, S]
    vh = vals.transpose(0, 2, 1, 3)                                          # [B, nq, S, D]
    scores = np.matmul(qh, kh).astype(np.float32) * np.float32(1.0 / np.sqrt(D))
    key_pos = np.arange(S, dtype=np.int32)
    if start_pos is None:
        visible = key_pos[None, :] <= np.arange(T, dtype=np.int32)[:, None]   # [T, S], trace-time constant
        scores = np.where(visible[None, None], scores, np.float32(-1e30))
    else:
        visible = tensor_apis.constant(key_pos)[None, :] <= start_pos[:, None]   # [1, S]
        scores = np.where(visible[None, None], scores, np.float32(-1e30))
    p = tensor_apis.softmax(scores).astype(x.dtype)       # one row kernel when compiled
    ctx = np.matmul(p, vh).transpose(0, 2, 1, 3).reshape(B, T, nq * D)
    return np.matmul(ctx, o_weight)
