"""Hugging Face checkpoints -> per-rank shards in this package's weight schema.

`convert_state_dict` maps the parameter names of the supported families (Llama / Qwen3 dense,
Qwen3-MoE, gpt-oss, Qwen3-Embedding) onto the schema documented in `weights.py`, transposes every
matrix into ``x @ W`` orientation, fuses q/k/v and gate/up, and slices the tensor- / expert-parallel
shard of `rank`.  `prepare_checkpoint` does that for every rank of a world size, reading
``*.safetensors`` lazily and writing ``shard_{rank}.safetensors``.

Reference parity: examples/models/qwen3/tensor_preparation.py:126-248 (Qwen3-MoE, experts sharded on
the intermediate axis), examples/models/gpt_oss/tensor_preparation.py:60-200 (interleaved gate/up,
biases, sinks, rank-0-only o_proj bias), examples/models/qwen3_embedding/prepare_weights.py:37-76.
Expert parallelism (`moe_parallel="ep"`, experts sharded on the expert axis) is new here.
"""

from __future__ import annotations

import glob
import json
import os
from typing import Callable, Dict, Iterable, Optional

import torch

from .config import ModelConfig
from .weights import kv_heads_for_rank, save_shard, shard_qkv

_FP4_VALUES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """MXFP4 (two e2m1 values per byte, one e8m0 scale per 32 values) -> dense tensor.
    blocks [..., G, 16] uint8, scales [..., G] uint8; returns [..., G * 32]."""
    lut = torch.tensor(_FP4_VALUES, dtype=torch.float32, device=blocks.device)
    lo = lut[(blocks & 0x0F).long()]
    hi = lut[(blocks >> 4).long()]
    vals = torch.stack([lo, hi], dim=-1).reshape(*blocks.shape[:-1], blocks.shape[-1] * 2)
    exp = (scales.to(torch.int32) - 127).to(torch.float32)
    out = vals * torch.pow(2.0, exp)[..., None]
    return out.reshape(*blocks.shape[:-2], -1).to(dtype)


class LazyCheckpoint:
    """Name -> tensor over the ``*.safetensors`` files of a directory, loaded on access."""

    def __init__(self, directory: str):
        from safetensors import safe_open

        self._open = safe_open
        self.files = sorted(glob.glob(os.path.join(directory, "*.safetensors")))
        if not self.files:
            raise FileNotFoundError(f"no *.safetensors under {directory}")
        self.index: Dict[str, str] = {}
        for f in self.files:
            with safe_open(f, framework="pt") as h:
                for k in h.keys():
                    self.index[k] = f

    def __contains__(self, name: str) -> bool:
        return name in self.index

    def keys(self) -> Iterable[str]:
        return self.index.keys()

    def __getitem__(self, name: str) -> torch.Tensor:
        with self._open(self.index[name], framework="pt") as h:
            return h.get_tensor(name)


def _cols(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[-1] // world
    return w[..., rank * n:(rank + 1) * n]


def _rows(w: torch.Tensor, rank: int, world: int, axis: int = 0) -> torch.Tensor:
    n = w.shape[axis] // world
    return w.narrow(axis, rank * n, n)


def convert_state_dict(cfg: ModelConfig, sd, rank: int = 0, world: int = 1, moe_parallel: str = "ep",
                       dtype=torch.bfloat16, family: Optional[str] = None) -> Dict[str, torch.Tensor]:
    """sd: mapping HF name -> tensor (a dict or a `LazyCheckpoint`)."""
    fam = family or ("gpt_oss" if cfg.attention_sinks else ("qwen3_moe" if cfg.is_moe else "dense"))
    pre = "model." if any(k.startswith("model.") for k in sd.keys()) else ""
    get: Callable[[str], torch.Tensor] = lambda n: sd[pre + n]
    T = lambda n: get(n).to(dtype).t().contiguous()          # nn.Linear stores [out, in]
    d, H = cfg.head_dim, cfg.hidden_size
    out: Dict[str, torch.Tensor] = {}
    out["tok_embedding"] = get("embed_tokens.weight").to(dtype).contiguous()
    out["norm_weight"] = get("norm.weight").to(dtype)
    lm_name = "lm_head.weight"
    if lm_name in sd:
        lm = sd[lm_name].to(dtype).t()
    else:                                                     # tied embeddings / embedding models
        lm = out["tok_embedding"].t()
    v_l = lm.shape[1] // world
    out["lm_head_weight"] = lm[:, rank * v_l:(rank + 1) * v_l].contiguous()
    nq_l = cfg.num_heads // world
    for i in range(cfg.num_layers):
        hp, p = f"layers.{i}.", f"layers.{i}."
        out[p + "qkv_weight"] = shard_qkv(T(hp + "self_attn.q_proj.weight"), T(hp + "self_attn.k_proj.weight"),
                                          T(hp + "self_attn.v_proj.weight"), cfg, rank, world)
        out[p + "o_weight"] = _rows(T(hp + "self_attn.o_proj.weight"), rank, world).contiguous()
        out[p + "input_layernorm_weight"] = get(hp + "input_layernorm.weight").to(dtype)
        out[p + "post_attention_layernorm_weight"] = get(hp + "post_attention_layernorm.weight").to(dtype)
        if cfg.qk_norm:
            out[p + "q_norm_weight"] = get(hp + "self_attn.q_norm.weight").to(dtype)
            out[p + "k_norm_weight"] = get(hp + "self_attn.k_norm.weight").to(dtype)
        if cfg.attn_bias:
            out[p + "qkv_bias"] = shard_qkv(get(hp + "self_attn.q_proj.bias").to(dtype),
                                            get(hp + "self_attn.k_proj.bias").to(dtype),
                                            get(hp + "self_attn.v_proj.bias").to(dtype), cfg, rank, world)
            bo = get(hp + "self_attn.o_proj.bias").to(dtype)
            out[p + "o_bias"] = bo if rank == 0 else torch.zeros_like(bo)   # added once by the reduction
        if cfg.attention_sinks:
            out[p + "sinks"] = get(hp + "self_attn.sinks").float()[rank * nq_l:(rank + 1) * nq_l].contiguous()
        if not cfg.is_moe:
            gate, up = T(hp + "mlp.gate_proj.weight"), T(hp + "mlp.up_proj.weight")
            out[p + "gate_up_weight"] = torch.cat([_cols(gate, rank, world), _cols(up, rank, world)], -1).contiguous()
            out[p + "down_weight"] = _rows(T(hp + "mlp.down_proj.weight"), rank, world).contiguous()
            continue
        E = cfg.num_experts
        if fam == "gpt_oss":
            out[p + "router_weight"] = T(hp + "mlp.router.weight")
            if cfg.router_bias:
                out[p + "router_bias"] = get(hp + "mlp.router.bias").to(dtype)
            name = hp + "mlp.experts.gate_up_proj"
            if pre + name in sd:
                gu = get(name).to(dtype)                                   # [E, H, 2I], gate / up interleaved
                dn = get(hp + "mlp.experts.down_proj").to(dtype)           # [E, I, H]
            else:                                                          # MXFP4 blocks + scales
                gu = dequant_mxfp4(get(name + "_blocks"), get(name + "_scales"), dtype).transpose(1, 2)
                dn = dequant_mxfp4(get(hp + "mlp.experts.down_proj_blocks"),
                                   get(hp + "mlp.experts.down_proj_scales"), dtype).transpose(1, 2)
            gate, up = gu[..., 0::2], gu[..., 1::2]
            gub = get(hp + "mlp.experts.gate_up_proj_bias").to(dtype) if cfg.expert_bias else None
            dnb = get(hp + "mlp.experts.down_proj_bias").to(dtype) if cfg.expert_bias else None
        else:
            out[p + "router_weight"] = T(hp + "mlp.gate.weight")
            gate = torch.stack([T(hp + f"mlp.experts.{e}.gate_proj.weight") for e in range(E)])   # [E, H, I]
            up = torch.stack([T(hp + f"mlp.experts.{e}.up_proj.weight") for e in range(E)])
            dn = torch.stack([T(hp + f"mlp.experts.{e}.down_proj.weight") for e in range(E)])     # [E, I, H]
            gub = dnb = None
        if moe_parallel == "ep":
            sl = slice(rank * (E // world), (rank + 1) * (E // world))
            out[p + "gate_up_weight"] = torch.cat([gate[sl], up[sl]], -1).contiguous()
            out[p + "down_weight"] = dn[sl].contiguous()
            if gub is not None:
                out[p + "gate_up_bias"] = torch.cat([gub[sl, 0::2], gub[sl, 1::2]], -1).contiguous()
                out[p + "down_bias"] = dnb[sl].contiguous()
        else:                                                              # reference layout: shard I
            out[p + "gate_up_weight"] = torch.cat([_cols(gate, rank, world), _cols(up, rank, world)], -1).contiguous()
            out[p + "down_weight"] = _rows(dn, rank, world, axis=1).contiguous()
            if gub is not None:
                out[p + "gate_up_bias"] = torch.cat([_cols(gub[:, 0::2], rank, world),
                                                     _cols(gub[:, 1::2], rank, world)], -1).contiguous()
                out[p + "down_bias"] = dnb if rank == 0 else torch.zeros_like(dnb)
    return out


def prepare_checkpoint(cfg: ModelConfig, model_dir: str, out_dir: str, world: int, moe_parallel: str = "ep",
                       family: Optional[str] = None) -> None:
    """Write ``shard_{rank}.safetensors`` for every rank plus ``prepared.json`` describing them."""
    sd = LazyCheckpoint(model_dir)
    os.makedirs(out_dir, exist_ok=True)
    for rank in range(world):
        save_shard(convert_state_dict(cfg, sd, rank, world, moe_parallel, family=family), out_dir, rank)
    with open(os.path.join(out_dir, "prepared.json"), "w") as f:
        json.dump({"model": cfg.name, "world_size": world, "moe_parallel": moe_parallel}, f)
