"""Kernel functions of the parallel-drafting (P-EAGLE) drafter.

One drafting step runs W rows per sequence at positions start_pos .. start_pos + W - 1: the tokens the target
accepted last step with their real tapped hidden states, then placeholder rows (a fixed token and the learnt
`mask_hidden`).  Row p pairs the embedding of token p + 1 with fc(target hidden states at p); the first ("fusion")
layer normalises the two halves separately, feeds their concatenation (2 H wide) to its attention and uses the
hidden half as the residual; the other layers are plain Llama layers.  The drafts are the arg-max over the
drafter's reduced vocabulary, mapped to target ids with the `d2t` offsets
(examples/models/gpt_oss/peagle/kernels/drafter.py:23-174 and drafter_layer.py in the reference)."""
import numpy as np

from nkipy_b200.core import tensor_apis

from llama_kernels.feedforward import swiglu_ffn
from llama_kernels.rmsnorm import rmsnorm
from llama_kernels.rope import rope_tables, rotate_halves


def fuse_inputs(token_ids, hidden3, is_mask, embed_tokens, fc_weight, mask_hidden, embed_norm, hidden_norm,
                norm_eps: float):
    """token_ids int32 [B, W]; hidden3 [B, W, 3 tH] (three tapped target layers); is_mask int32 [B, W] (1 =
    placeholder row).  Returns (residual [B, W, H], first-layer input [B, W, 2 H])."""
    emb = np.take(embed_tokens, token_ids, axis=0)
    h3 = np.where(is_mask[:, :, None] != 0, mask_hidden[None, None, :], hidden3)
    hid = np.matmul(h3, fc_weight)
    fused = np.concatenate([rmsnorm(emb, embed_norm, norm_eps), rmsnorm(hid, hidden_norm, norm_eps)], axis=-1)
    return hid, fused


def window_attention(h, qkv_weight, o_weight, cache_k, cache_v, start_pos, *, n_heads: int, n_kv_heads: int,
                     head_dim: int, rope_theta: float):
    """Causal attention of W rows at positions start_pos + 0 .. W - 1 (start_pos int32 [1]) over a dense cache
    [B, S_max, nkv, D] that the kernel updates in place; rows past a query's position stay hidden, so rejected rows
    of an earlier step are simply overwritten."""
    B, W, _ = h.shape
    S = cache_k.shape[1]
    nq, nkv, D = n_heads, n_kv_heads, head_dim
    qkv = np.matmul(h, qkv_weight)
    q, k, v = np.split(qkv, [nq * D, (nq + nkv) * D], axis=-1)
    q, k, v = q.reshape(B, W, nq, D), k.reshape(B, W, nkv, D), v.reshape(B, W, nkv, D)
    cos, sin = rope_tables(D, S, rope_theta)
    cos_c, sin_c = tensor_apis.constant(cos), tensor_apis.constant(sin)
    rows_q, rows_k = [], []
    for i in range(W):                                           # W is small (twice the draft length)
        pos = start_pos + np.int32(i)
        c, s = cos_c[pos][None, :, None, :], sin_c[pos][None, :, None, :]
        rows_q.append(rotate_halves(q[:, i:i + 1], c, s))
        ki = rotate_halves(k[:, i:i + 1], c, s)
        rows_k.append(ki)
        cache_k[:, pos] = ki
        cache_v[:, pos] = v[:, i:i + 1]
    q = np.concatenate(rows_q, axis=1)
    rep = nq // nkv
    keys = np.repeat(cache_k, rep, axis=2) if rep > 1 else cache_k
    vals = np.repeat(cache_v, rep, axis=2) if rep > 1 else cache_v
    scores = np.matmul(q.transpose(0, 2, 1, 3), keys.transpose(0, 2, 3, 1)).astype(np.float32)
    scores = scores * np.float32(1.0 / np.sqrt(D))                                  # [B, nq, W, S]
    key_pos = tensor_apis.constant(np.arange(S, dtype=np.int32))[None, :]           # [1, S]
    q_pos = start_pos[:, None] + tensor_apis.constant(np.arange(W, dtype=np.int32))[:, None]   # [W, 1]
    scores = np.where((key_pos <= q_pos)[None, None], scores, np.float32(-1e30))
    p = tensor_apis.softmax(scores).astype(h.dtype)
    ctx = np.matmul(p, vals.transpose(0, 2, 1, 3)).transpose(0, 2, 1, 3).reshape(B, W, nq * D)
    return np.matmul(ctx, o_weight)


def fusion_layer(hid, fused, start_pos, qkv_weight, o_weight, gate_up_weight, down_weight, post_norm, cache_k, cache_v,
                 n_heads, n_kv_heads, head_dim, rope_theta, norm_eps):
    """First drafter layer: attention over the 2 H-wide fused input, the hidden half as the residual."""
    x = hid + window_attention(fused, qkv_weight, o_weight, cache_k, cache_v, start_pos, n_heads=n_heads,
                               n_kv_heads=n_kv_heads, head_dim=head_dim, rope_theta=rope_theta)
    return x + swiglu_ffn(rmsnorm(x, post_norm, norm_eps), gate_up_weight, down_weight)


def drafter_layer(x, start_pos, qkv_weight, o_weight, gate_up_weight, down_weight, input_norm, post_norm, cache_k,
                  cache_v, n_heads, n_kv_heads, head_dim, rope_theta, norm_eps):
    """The other drafter layers: a Llama layer over the same window of rows."""
    x = x + window_attention(rmsnorm(x, input_norm, norm_eps), qkv_weight, o_weight, cache_k, cache_v, start_pos,
                             n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, rope_theta=rope_theta)
    return x + swiglu_ffn(rmsnorm(x, post_norm, norm_eps), gate_up_weight, down_weight)


def draft_tokens(x, final_norm, lm_head, d2t, norm_eps: float):
    """x [B, W, H]; lm_head [H, V_draft]; d2t int32 [V_draft] (offset from a draft-vocabulary id to the target id).
    Returns int32 [B, W]: the proposed target-vocabulary token of every row."""
    logits = np.matmul(rmsnorm(x, final_norm, norm_eps), lm_head).astype(np.float32)
    idx = np.argmax(logits, axis=-1).astype(np.int32)
    return idx + np.take(d2t, idx, axis=0)
