"""One decoder layer as a kernel function: norm, attention with its cache update, residual, norm, SwiGLU,
residual.  `prefill_layer` and `decode_layer` differ only in how positions reach the attention block
(examples/models/qwen3/kernels/transformer_layer.py:17-115 in the reference has the same split)."""
from .attention import attention_block
from .feedforward import swiglu_ffn
from .rmsnorm import rmsnorm


def _layer(x, start_pos, qkv_weight, o_weight, gate_up_weight, down_weight, input_norm, post_norm, cache_k, cache_v,
           n_heads, n_kv_heads, head_dim, rope_theta, norm_eps):
    h = rmsnorm(x, input_norm, norm_eps)
    x = x + attention_block(h, qkv_weight, o_weight, cache_k, cache_v, start_pos, n_heads=n_heads,
                            n_kv_heads=n_kv_heads, head_dim=head_dim, rope_theta=rope_theta, norm_eps=norm_eps)
    h = rmsnorm(x, post_norm, norm_eps)
    return x + swiglu_ffn(h, gate_up_weight, down_weight)


def prefill_layer(x, qkv_weight, o_weight, gate_up_weight, down_weight, input_norm, post_norm, cache_k, cache_v,
                  n_heads, n_kv_heads, head_dim, rope_theta, norm_eps):
    return _layer(x, None, qkv_weight, o_weight, gate_up_weight, down_weight, input_norm, post_norm, cache_k,
                  cache_v, n_heads, n_kv_heads, head_dim, rope_theta, norm_eps)


def decode_layer(x, start_pos, qkv_weight, o_weight, gate_up_weight, down_weight, input_norm, post_norm, cache_k,
                 cache_v, n_heads, n_kv_heads, head_dim, rope_theta, norm_eps):
    return _layer(x, start_pos, qkv_weight, o_weight, gate_up_weight, down_weight, input_norm, post_norm, cache_k,
                  cache_v, n_heads, n_kv_heads, head_dim, rope_theta, norm_eps)
