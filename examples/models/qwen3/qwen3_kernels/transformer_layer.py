"""One Qwen3-MoE decoder layer as a kernel function: norm, attention with QK-norm and its cache update, residual,
norm, routed feed-forward, residual (examples/models/qwen3/kernels/transformer_layer.py:16-115 in the reference)."""
from llama_kernels.attention import attention_block
from llama_kernels.rmsnorm import rmsnorm

from .moe import moe_ffn


def _layer(x, start_pos, qkv_weight, o_weight, q_norm, k_norm, router_weight, gate_up_weight, down_weight, input_norm,
           post_norm, cache_k, cache_v, n_heads, n_kv_heads, head_dim, rope_theta, norm_eps, top_k):
    h = rmsnorm(x, input_norm, norm_eps)
    x = x + attention_block(h, qkv_weight, o_weight, cache_k, cache_v, start_pos, n_heads=n_heads,
                            n_kv_heads=n_kv_heads, head_dim=head_dim, rope_theta=rope_theta, q_norm=q_norm,
                            k_norm=k_norm, norm_eps=norm_eps)
    h = rmsnorm(x, post_norm, norm_eps)
    return x + moe_ffn(h, router_weight, gate_up_weight, down_weight, top_k)


def prefill_layer(x, qkv_weight, o_weight, q_norm, k_norm, router_weight, gate_up_weight, down_weight, input_norm,
                  post_norm, cache_k, cache_v, n_heads, n_kv_heads, head_dim, rope_theta, norm_eps, top_k):
    return _layer(x, None, qkv_weight, o_weight, q_norm, k_norm, router_weight, gate_up_weight, down_weight,
                  input_norm, post_norm, cache_k, cache_v, n_heads, n_kv_heads, head_dim, rope_theta, norm_eps, top_k)


def decode_layer(x, start_pos, qkv_weight, o_weight, q_norm, k_norm, router_weight, gate_up_weight, down_weight,
                 input_norm, post_norm, cache_k, cache_v, n_heads, n_kv_heads, head_dim, rope_theta, norm_eps, top_k):
    return _layer(x, start_pos, qkv_weight, o_weight, q_norm, k_norm, router_weight, gate_up_weight, down_weight,
                  input_norm, post_norm, cache_k, cache_v, n_heads, n_kv_heads, head_dim, rope_theta, norm_eps, top_k)
