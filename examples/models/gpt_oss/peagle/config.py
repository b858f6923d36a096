"""Drafter shape for the gpt-oss P-EAGLE example (reference: examples/models/gpt_oss/peagle/config.py:12-83)."""
from nkipy_b200.models.speculative import EagleConfig


def get_eagle_config(target_cfg, num_draft_tokens: int = 3, draft_vocab_size: int = 32000) -> EagleConfig:
    return EagleConfig(hidden_size=target_cfg.hidden_size, target_hidden_size=target_cfg.hidden_size, num_layers=4,
                       num_heads=target_cfg.num_heads, num_kv_heads=target_cfg.num_kv_heads,
                       head_dim=target_cfg.head_dim, intermediate_size=4 * target_cfg.hidden_size,
                       draft_vocab_size=min(draft_vocab_size, target_cfg.vocab_size),
                       vocab_size=target_cfg.vocab_size, ptd_token_id=0, num_draft_tokens=num_draft_tokens,
                       rms_eps=target_cfg.rms_eps, rope_theta=target_cfg.rope_theta,
                       max_position=target_cfg.max_position)
