"""Model shape of the Qwen3 MoE example (reference: examples/models/qwen3/config.py:31-46 reads the
same fields from the Hugging Face config)."""
import json
import os

from nkipy_b200.models.config import ModelConfig, qwen3_30b_a3b


def get_config(model_dir=None) -> ModelConfig:
    cfg = qwen3_30b_a3b()
    if model_dir and os.path.exists(os.path.join(model_dir, "config.json")):
        with open(os.path.join(model_dir, "config.json")) as f:
            hf = json.load(f)
        cfg.vocab_size = hf.get("vocab_size", cfg.vocab_size)
        cfg.hidden_size = hf.get("hidden_size", cfg.hidden_size)
        cfg.num_layers = hf.get("num_hidden_layers", cfg.num_layers)
        cfg.num_heads = hf.get("num_attention_heads", cfg.num_heads)
        cfg.num_kv_heads = hf.get("num_key_value_heads", cfg.num_kv_heads)
        cfg.head_dim = hf.get("head_dim", cfg.head_dim)
        cfg.num_experts = hf.get("num_experts", cfg.num_experts)
        cfg.top_k = hf.get("num_experts_per_tok", cfg.top_k)
        cfg.moe_intermediate_size = hf.get("moe_intermediate_size", cfg.moe_intermediate_size)
        cfg.rope_theta = hf.get("rope_theta", cfg.rope_theta)
        cfg.rms_eps = hf.get("rms_norm_eps", cfg.rms_eps)
    return cfg
