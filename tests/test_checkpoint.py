"""HF-layout state dicts -> per-rank shards: the converter must agree with `random_weights`, which
slices shards of the same full model independently."""
import os

import pytest
import torch

from nkipy_b200.models import config as C
from nkipy_b200.models.checkpoint import LazyCheckpoint, convert_state_dict, dequant_mxfp4, prepare_checkpoint
from nkipy_b200.models.weights import load_shard, random_weights


def _to_hf(cfg, w):
    """Inverse mapping of the schema for a world-size-1 weight dict."""
    d = cfg.head_dim
    sd = {"model.embed_tokens.weight": w["tok_embedding"], "model.norm.weight": w["norm_weight"],
          "lm_head.weight": w["lm_head_weight"].t().contiguous()}
    qs, ks = cfg.num_heads * d, cfg.num_kv_heads * d
    for i in range(cfg.num_layers):
        p, h = f"layers.{i}.", f"model.layers.{i}."
        qkv = w[p + "qkv_weight"]
        sd[h + "self_attn.q_proj.weight"] = qkv[:, :qs].t().contiguous()
        sd[h + "self_attn.k_proj.weight"] = qkv[:, qs:qs + ks].t().contiguous()
        sd[h + "self_attn.v_proj.weight"] = qkv[:, qs + ks:].t().contiguous()
        sd[h + "self_attn.o_proj.weight"] = w[p + "o_weight"].t().contiguous()
        sd[h + "input_layernorm.weight"] = w[p + "input_layernorm_weight"]
        sd[h + "post_attention_layernorm.weight"] = w[p + "post_attention_layernorm_weight"]
        if cfg.qk_norm:
            sd[h + "self_attn.q_norm.weight"] = w[p + "q_norm_weight"]
            sd[h + "self_attn.k_norm.weight"] = w[p + "k_norm_weight"]
        if cfg.attn_bias:
            b = w[p + "qkv_bias"]
            sd[h + "self_attn.q_proj.bias"], sd[h + "self_attn.k_proj.bias"] = b[:qs], b[qs:qs + ks]
            sd[h + "self_attn.v_proj.bias"] = b[qs + ks:]
            sd[h + "self_attn.o_proj.bias"] = w[p + "o_bias"]
        if cfg.attention_sinks:
            sd[h + "self_attn.sinks"] = w[p + "sinks"]
        if not cfg.is_moe:
            gu = w[p + "gate_up_weight"]
            I = gu.shape[1] // 2
            sd[h + "mlp.gate_proj.weight"] = gu[:, :I].t().contiguous()
            sd[h + "mlp.up_proj.weight"] = gu[:, I:].t().contiguous()
            sd[h + "mlp.down_proj.weight"] = w[p + "down_weight"].t().contiguous()
        elif cfg.attention_sinks:       # gpt-oss: fused, interleaved experts
            gu = w[p + "gate_up_weight"]                       # [E, H, 2I] gate | up
            I = gu.shape[-1] // 2
            inter = torch.empty_like(gu)
            inter[..., 0::2], inter[..., 1::2] = gu[..., :I], gu[..., I:]
            sd[h + "mlp.experts.gate_up_proj"] = inter
            sd[h + "mlp.experts.down_proj"] = w[p + "down_weight"]
            gb = w[p + "gate_up_bias"]
            gbi = torch.empty_like(gb)
            gbi[:, 0::2], gbi[:, 1::2] = gb[:, :I], gb[:, I:]
            sd[h + "mlp.experts.gate_up_proj_bias"] = gbi
            sd[h + "mlp.experts.down_proj_bias"] = w[p + "down_bias"]
            sd[h + "mlp.router.weight"] = w[p + "router_weight"].t().contiguous()
            sd[h + "mlp.router.bias"] = w[p + "router_bias"]
        else:
            gu, dn = w[p + "gate_up_weight"], w[p + "down_weight"]
            I = gu.shape[-1] // 2
            sd[h + "mlp.gate.weight"] = w[p + "router_weight"].t().contiguous()
            for e in range(cfg.num_experts):
                sd[h + f"mlp.experts.{e}.gate_proj.weight"] = gu[e, :, :I].t().contiguous()
                sd[h + f"mlp.experts.{e}.up_proj.weight"] = gu[e, :, I:].t().contiguous()
                sd[h + f"mlp.experts.{e}.down_proj.weight"] = dn[e].t().contiguous()
    return sd


CONFIGS = {
    "dense": lambda: C.tiny(num_heads=4, num_kv_heads=2),
    "qwen3_moe": lambda: C.tiny(num_heads=4, num_kv_heads=2, qk_norm=True, num_experts=8, top_k=2,
                                moe_intermediate_size=64, intermediate_size=0),
    "gpt_oss": lambda: C.tiny(num_heads=4, num_kv_heads=2, attn_bias=True, attention_sinks=True, num_experts=4,
                              top_k=2, moe_intermediate_size=64, intermediate_size=0, router_bias=True,
                              expert_bias=True, router_mode="topk_softmax", swiglu_limit=7.0),
}


@pytest.mark.parametrize("kind", list(CONFIGS))
@pytest.mark.parametrize("world,moe_parallel", [(1, "ep"), (2, "ep"), (2, "tp")])
def test_converter_matches_random_weights(kind, world, moe_parallel):
    cfg = CONFIGS[kind]()
    sd = _to_hf(cfg, random_weights(cfg, 0, 1, seed=3))
    for rank in range(world):
        got = convert_state_dict(cfg, sd, rank, world, moe_parallel)
        want = random_weights(cfg, rank, world, seed=3, moe_parallel=moe_parallel)
        assert set(got) == set(want), set(got) ^ set(want)
        for k in want:
            assert got[k].shape == want[k].shape, k
            assert torch.equal(got[k].float(), want[k].float()), k


def test_prepare_checkpoint_roundtrip(tmp_path):
    from safetensors.torch import save_file

    cfg = CONFIGS["dense"]()
    sd = _to_hf(cfg, random_weights(cfg, 0, 1, seed=4))
    src, dst = tmp_path / "hf", tmp_path / "out"
    os.makedirs(src)
    keys = sorted(sd)
    save_file({k: sd[k].contiguous() for k in keys[:len(keys) // 2]}, str(src / "model-00001-of-00002.safetensors"))
    save_file({k: sd[k].contiguous() for k in keys[len(keys) // 2:]}, str(src / "model-00002-of-00002.safetensors"))
    assert "lm_head.weight" in LazyCheckpoint(str(src))
    prepare_checkpoint(cfg, str(src), str(dst), world=2)
    for rank in range(2):
        got = load_shard(str(dst), rank)
        want = random_weights(cfg, rank, 2, seed=4)
        assert all(torch.equal(got[k].float(), want[k].float()) for k in want)


def test_mxfp4_dequant():
    blocks = torch.tensor([[[0x21, 0xF8] + [0] * 14]], dtype=torch.uint8)      # nibbles: 1,2 | 8,15
    scales = torch.tensor([[128]], dtype=torch.uint8)                           # x 2
    out = dequant_mxfp4(blocks, scales, torch.float32)
    assert out.shape == (1, 32)
    assert out[0, :4].tolist() == [1.0, 2.0, -0.0, -12.0]
