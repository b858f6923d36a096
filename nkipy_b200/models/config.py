"""Model configurations.

One dataclass covers the decoder families of the reference examples: dense
Llama-style (tests/kernels/llama_decoder_dynamo.py, qwen3_embedding), Qwen3 MoE
(examples/models/qwen3/config.py:12-46) and gpt-oss
(examples/models/gpt_oss/config.py:14-68: alternating sliding-window layers,
attention sinks, biases, clamped SwiGLU, YaRN RoPE).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import List, Optional


@dataclass
class ModelConfig:
    name: str = "llama"
    vocab_size: int = 128256
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 14336
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_position: int = 8192
    qk_norm: bool = False                 # per-head RMSNorm on q and k (Qwen3)
    attn_bias: bool = False               # qkv / o biases (gpt-oss)
    causal: bool = True
    # MoE (num_experts == 0 -> dense SwiGLU FFN)
    num_experts: int = 0
    top_k: int = 0
    moe_intermediate_size: int = 0
    router_mode: str = "softmax_topk"     # or "topk_softmax" (gpt-oss)
    router_bias: bool = False
    expert_bias: bool = False
    # gpt-oss attention features
    sliding_window: int = 0
    layer_types: Optional[List[str]] = None   # "full_attention" | "sliding_attention" per layer
    attention_sinks: bool = False
    swiglu_limit: float = 0.0             # > 0 selects the clamped (up + 1) * gate * sigmoid(alpha * gate) form
    swiglu_alpha: float = 1.702
    # YaRN
    rope_scaling_factor: float = 1.0
    rope_original_max_position: int = 0
    rope_beta_fast: float = 32.0
    rope_beta_slow: float = 1.0
    block_size: int = 32

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def window_for_layer(self, layer: int) -> int:
        if self.sliding_window <= 0:
            return 0
        if self.layer_types is None:
            return self.sliding_window
        return self.sliding_window if self.layer_types[layer] == "sliding_attention" else 0

    def scaled(self, **overrides) -> "ModelConfig":
        return replace(self, **overrides)

    def shard_shapes(self, n: int) -> "ModelConfig":
        """The configuration whose full model has the per-rank shapes of this one under n-way tensor
        (and expert) parallelism: 1/n of the heads, of the FFN width, of the experts and of the
        vocabulary.  Used to time the kernels of one rank of an n-GPU job on a single GPU."""
        if n <= 1:
            return self
        return replace(
            self, name=f"{self.name}-shard{n}", num_heads=max(1, self.num_heads // n),
            num_kv_heads=max(1, self.num_kv_heads // n), intermediate_size=self.intermediate_size // n,
            num_experts=self.num_experts // n if self.is_moe else 0,
            top_k=max(1, self.top_k // n) if self.is_moe else 0,      # same (token, expert) pairs per rank
            vocab_size=self.vocab_size // n)

    def param_count(self) -> int:
        h = self.hidden_size
        attn = h * (self.q_size + 2 * self.kv_size) + self.q_size * h
        if self.is_moe:
            ffn = self.num_experts * 3 * h * self.moe_intermediate_size + h * self.num_experts
        else:
            ffn = 3 * h * self.intermediate_size
        return self.num_layers * (attn + ffn + 2 * h) + 2 * self.vocab_size * h + h


def llama3_8b(**kw) -> ModelConfig:
    """Llama-3-8B-shaped dense decoder."""
    return ModelConfig(name="llama3-8b", **kw)


def qwen3_30b_a3b(**kw) -> ModelConfig:
    """Qwen3-30B-A3B-shaped MoE decoder (128 experts, top-8, expert FFN 768)."""
    base = dict(name="qwen3-30b-a3b", vocab_size=151936, hidden_size=2048, num_layers=48, num_heads=32,
                num_kv_heads=4, head_dim=128, intermediate_size=0, rms_eps=1e-6, rope_theta=1e6,
                max_position=40960, qk_norm=True, num_experts=128, top_k=8, moe_intermediate_size=768)
    base.update(kw)
    return ModelConfig(**base)


def gpt_oss_20b(**kw) -> ModelConfig:
    """gpt-oss-20b-shaped MoE decoder (32 experts, top-4, sliding window 128 on alternating layers)."""
    n = kw.get("num_layers", 24)
    base = dict(name="gpt-oss-20b", vocab_size=201088, hidden_size=2880, num_layers=n, num_heads=64,
                num_kv_heads=8, head_dim=64, intermediate_size=0, rms_eps=1e-5, rope_theta=150000.0,
                max_position=131072, attn_bias=True, num_experts=32, top_k=4, moe_intermediate_size=2880,
                router_mode="topk_softmax", router_bias=True, expert_bias=True, sliding_window=128,
                layer_types=["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(n)],
                attention_sinks=True, swiglu_limit=7.0, swiglu_alpha=1.702, rope_scaling_factor=32.0,
                rope_original_max_position=4096)
    base.update(kw)
    return ModelConfig(**base)


def qwen3_embedding(size: str = "0.6b", **kw) -> ModelConfig:
    """Qwen3-Embedding-shaped dense encoder-style decoder (examples/models/qwen3_embedding/config.py:15-112)."""
    presets = {
        "0.6b": dict(hidden_size=1024, num_layers=28, num_heads=16, num_kv_heads=8, intermediate_size=3072),
        "8b": dict(hidden_size=4096, num_layers=36, num_heads=32, num_kv_heads=8, intermediate_size=12288),
    }
    base = dict(name=f"qwen3-embedding-{size}", vocab_size=151669, head_dim=128, rms_eps=1e-6, rope_theta=1e6,
                max_position=32768, qk_norm=True)
    base.update(presets[size])
    base.update(kw)
    return ModelConfig(**base)


def tiny(**kw) -> ModelConfig:
    """Small dense config for unit tests and the smoke run."""
    base = dict(name="tiny", vocab_size=512, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                head_dim=64, intermediate_size=512, max_position=512)
    base.update(kw)
    return ModelConfig(**base)


def yarn_inv_freq(cfg: ModelConfig):
    """(inv_freq [head_dim/2], attention scaling) for the configured RoPE; plain RoPE when
    rope_scaling_factor == 1 (YaRN per examples/models/gpt_oss/config.py:64-68)."""
    import torch

    d = cfg.head_dim
    base = cfg.rope_theta
    freq = base ** (torch.arange(0, d, 2, dtype=torch.float64) / d)
    if cfg.rope_scaling_factor <= 1.0:
        return (1.0 / freq), 1.0
    factor = cfg.rope_scaling_factor
    orig = cfg.rope_original_max_position
    concentration = 0.1 * math.log(factor) + 1.0
    d_half = d / 2
    low = d_half * math.log(orig / (cfg.rope_beta_fast * 2 * math.pi)) / math.log(base)
    high = d_half * math.log(orig / (cfg.rope_beta_slow * 2 * math.pi)) / math.log(base)
    interpolation = 1.0 / (factor * freq)
    extrapolation = 1.0 / freq
    ramp = (torch.arange(d_half, dtype=torch.float64) - low) / (high - low)
    mask = 1 - ramp.clamp(0, 1)
    inv_freq = interpolation * (1 - mask) + extrapolation * mask
    return inv_freq, concentration
