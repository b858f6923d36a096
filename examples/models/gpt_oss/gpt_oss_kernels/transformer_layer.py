"""One gpt-oss decoder layer as a kernel function; `window` (0 or the sliding window) is a compile-time number, so
the sliding and the full-attention layers are two graphs."""
from llama_kernels.rmsnorm import rmsnorm

from .attention import attention_block
from .moe import moe_ffn


def _layer(x, start_pos, qkv_weight, qkv_bias, o_weight, o_bias, sinks, router_weight, router_bias, gate_up_weight,
           gate_up_bias, down_weight, down_bias, input_norm, post_norm, cos, sin, cache_k, cache_v, n_heads, n_kv_heads,
           head_dim, norm_eps, top_k, limit, alpha, window):
    h = rmsnorm(x, input_norm, norm_eps)
    x = x + attention_block(h, qkv_weight, qkv_bias, o_weight, o_bias, sinks, cos, sin, cache_k, cache_v, start_pos,
                            n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, window=window)
    h = rmsnorm(x, post_norm, norm_eps)
    return x + moe_ffn(h, router_weight, router_bias, gate_up_weight, gate_up_bias, down_weight, down_bias, top_k,
                       limit, alpha)


def prefill_layer(x, qkv_weight, qkv_bias, o_weight, o_bias, sinks, router_weight, router_bias, gate_up_weight,
                  gate_up_bias, down_weight, down_bias, input_norm, post_norm, cos, sin, cache_k, cache_v, n_heads,
                  n_kv_heads, head_dim, norm_eps, top_k, limit, alpha, window):
    return _layer(x, None, qkv_weight, qkv_bias, o_weight, o_bias, sinks, router_weight, router_bias, gate_up_weight,
                  gate_up_bias, down_weight, down_bias, input_norm, post_norm, cos, sin, cache_k, cache_v, n_heads,
                  n_kv_heads, head_dim, norm_eps, top_k, limit, alpha, window)


def decode_layer(x, start_pos, qkv_weight, qkv_bias, o_weight, o_bias, sinks, router_weight, router_bias,
                 gate_up_weight, gate_up_bias, down_weight, down_bias, input_norm, post_norm, cos, sin, cache_k,
                 cache_v, n_heads, n_kv_heads, head_dim, norm_eps, top_k, limit, alpha, window):
    return _layer(x, start_pos, qkv_weight, qkv_bias, o_weight, o_bias, sinks, router_weight, router_bias,
                  gate_up_weight, gate_up_bias, down_weight, down_bias, input_norm, post_norm, cos, sin, cache_k,
                  cache_v, n_heads, n_kv_heads, head_dim, norm_eps, top_k, limit, alpha, window)
