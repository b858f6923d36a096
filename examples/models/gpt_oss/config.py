"""Model shape of the gpt-oss example (reference: examples/models/gpt_oss/config.py:20-89)."""
import json
import os

from nkipy_b200.models.config import ModelConfig, gpt_oss_20b


def get_config(model_dir=None) -> ModelConfig:
    cfg = gpt_oss_20b()
    if model_dir and os.path.exists(os.path.join(model_dir, "config.json")):
        with open(os.path.join(model_dir, "config.json")) as f:
            hf = json.load(f)
        cfg.vocab_size = hf.get("vocab_size", cfg.vocab_size)
        cfg.hidden_size = hf.get("hidden_size", cfg.hidden_size)
        cfg.num_layers = hf.get("num_hidden_layers", cfg.num_layers)
        cfg.num_heads = hf.get("num_attention_heads", cfg.num_heads)
        cfg.num_kv_heads = hf.get("num_key_value_heads", cfg.num_kv_heads)
        cfg.head_dim = hf.get("head_dim", cfg.head_dim)
        cfg.num_experts = hf.get("num_local_experts", cfg.num_experts)
        cfg.top_k = hf.get("num_experts_per_tok", cfg.top_k)
        cfg.moe_intermediate_size = hf.get("intermediate_size", cfg.moe_intermediate_size)
        cfg.sliding_window = hf.get("sliding_window", cfg.sliding_window)
    return cfg
