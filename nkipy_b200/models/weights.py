"""Weight preparation: per-rank shards in the reference's safetensors schema.

Key names and orientation follow the reference converters
(examples/models/qwen3/tensor_preparation.py:126-248,
examples/models/qwen3_embedding/prepare_weights.py:37-76): every matrix is
stored in ``x @ W`` orientation,

    tok_embedding [V, H]            norm_weight [H]         lm_head_weight [H, V/tp]
    layers.{i}.qkv_weight [H, (nq + 2 nkv) d / tp]          layers.{i}.o_weight [nq d / tp, H]
    layers.{i}.input_layernorm_weight [H]                   layers.{i}.post_attention_layernorm_weight [H]
    dense:  layers.{i}.gate_up_weight [H, 2 I / tp]  (gate | up)   layers.{i}.down_weight [I / tp, H]
    MoE:    layers.{i}.router_weight [H, E]
            layers.{i}.gate_up_weight [E_local, H, 2 I_local]      layers.{i}.down_weight [E_local, I_local, H]
    Qwen3:  layers.{i}.q_norm_weight [d], k_norm_weight [d]
    gpt-oss: qkv_bias, o_bias, router_bias, gate_up_bias, down_bias, sinks [nq / tp]

Column-parallel tensors (qkv, gate_up, lm_head) are split on their output axis,
row-parallel ones (o, down) on their input axis; KV heads are replicated when a
rank would own less than one head (tensor_preparation.py:82-91).  The reference
shards MoE experts on the intermediate axis (every rank holds all experts);
`moe_parallel="ep"` shards the expert axis instead (new here).
"""

from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from .config import ModelConfig


def _normal(shape, std, seed, device, dtype=torch.bfloat16):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(dtype)


def kv_heads_for_rank(cfg: ModelConfig, rank: int, world: int):
    """(first kv head, number of kv heads) owned by `rank`; heads are replicated when world > num_kv_heads."""
    if cfg.num_kv_heads >= world:
        n = cfg.num_kv_heads // world
        return rank * n, n
    rep = world // cfg.num_kv_heads
    return rank // rep, 1


def shard_qkv(w_q, w_k, w_v, cfg: ModelConfig, rank: int, world: int):
    """Fuse this rank's q / k / v columns: [H, (nq_l + 2 nkv_l) d]."""
    d = cfg.head_dim
    nq_l = cfg.num_heads // world
    kv0, nkv_l = kv_heads_for_rank(cfg, rank, world)
    q = w_q[..., rank * nq_l * d:(rank + 1) * nq_l * d]
    k = w_k[..., kv0 * d:(kv0 + nkv_l) * d]
    v = w_v[..., kv0 * d:(kv0 + nkv_l) * d]
    return torch.cat([q, k, v], dim=-1).contiguous()


def random_weights(cfg: ModelConfig, rank: int = 0, world: int = 1, device="cpu", seed: int = 0, std: float = 0.02,
                   moe_parallel: str = "ep", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Random-init weights ~ N(0, std) for `rank` of `world`, in the schema above.  The
    full tensor of every parameter is generated from a per-parameter seed and then
    sliced, so all ranks of any world size see shards of the same model."""
    H, d, V = cfg.hidden_size, cfg.head_dim, cfg.vocab_size
    out: Dict[str, torch.Tensor] = {}
    sid = [seed * 100003]

    def nxt():
        sid[0] += 1
        return sid[0]

    out["tok_embedding"] = _normal((V, H), std, nxt(), device, dtype)
    out["norm_weight"] = torch.ones(H, dtype=dtype, device=device)
    v_l = V // world
    lm = _normal((H, V), std, nxt(), device, dtype)
    out["lm_head_weight"] = lm[:, rank * v_l:(rank + 1) * v_l].contiguous()
    del lm
    for i in range(cfg.num_layers):
        p = f"layers.{i}."
        wq = _normal((H, cfg.q_size), std, nxt(), device, dtype)
        wk = _normal((H, cfg.kv_size), std, nxt(), device, dtype)
        wv = _normal((H, cfg.kv_size), std, nxt(), device, dtype)
        out[p + "qkv_weight"] = shard_qkv(wq, wk, wv, cfg, rank, world)
        del wq, wk, wv
        nq_l = cfg.num_heads // world
        wo = _normal((cfg.q_size, H), std, nxt(), device, dtype)
        out[p + "o_weight"] = wo[rank * nq_l * d:(rank + 1) * nq_l * d].contiguous()
        del wo
        out[p + "input_layernorm_weight"] = torch.ones(H, dtype=dtype, device=device)
        out[p + "post_attention_layernorm_weight"] = torch.ones(H, dtype=dtype, device=device)
        if cfg.qk_norm:
            out[p + "q_norm_weight"] = torch.ones(d, dtype=dtype, device=device)
            out[p + "k_norm_weight"] = torch.ones(d, dtype=dtype, device=device)
        if cfg.attn_bias:
            bq = _normal((cfg.q_size,), std, nxt(), device, dtype)
            bk = _normal((cfg.kv_size,), std, nxt(), device, dtype)
            bv = _normal((cfg.kv_size,), std, nxt(), device, dtype)
            out[p + "qkv_bias"] = shard_qkv(bq, bk, bv, cfg, rank, world)
            bo = _normal((H,), std, nxt(), device, dtype)
            # row-parallel bias is applied once: only rank 0 keeps it (gpt_oss/tensor_preparation.py:131-133)
            out[p + "o_bias"] = bo if rank == 0 else torch.zeros_like(bo)
        if cfg.attention_sinks:
            s = _normal((cfg.num_heads,), 1.0, nxt(), device, torch.float32)
            out[p + "sinks"] = s[rank * nq_l:(rank + 1) * nq_l].contiguous()
        if not cfg.is_moe:
            I = cfg.intermediate_size
            i_l = I // world
            wg = _normal((H, I), std, nxt(), device, dtype)
            wu = _normal((H, I), std, nxt(), device, dtype)
            out[p + "gate_up_weight"] = torch.cat(
                [wg[:, rank * i_l:(rank + 1) * i_l], wu[:, rank * i_l:(rank + 1) * i_l]], dim=-1).contiguous()
            del wg, wu
            wd = _normal((I, H), std, nxt(), device, dtype)
            out[p + "down_weight"] = wd[rank * i_l:(rank + 1) * i_l].contiguous()
            del wd
        else:
            E, I = cfg.num_experts, cfg.moe_intermediate_size
            out[p + "router_weight"] = _normal((H, E), std, nxt(), device, dtype)
            if cfg.router_bias:
                out[p + "router_bias"] = _normal((E,), std, nxt(), device, dtype)
            if moe_parallel == "ep":
                e_l, i_l = E // world, I
                e0, i0 = rank * e_l, 0
            else:
                e_l, i_l = E, I // world
                e0, i0 = 0, rank * i_l
            gs, us, ds = nxt(), nxt(), nxt()
            gu = torch.empty((e_l, H, 2 * i_l), dtype=dtype, device=device)
            dn = torch.empty((e_l, i_l, H), dtype=dtype, device=device)
            for e in range(e_l):
                ge = e0 + e
                wg = _normal((H, I), std, gs * 1009 + ge, device, dtype)
                wu = _normal((H, I), std, us * 1009 + ge, device, dtype)
                wd = _normal((I, H), std, ds * 1009 + ge, device, dtype)
                gu[e, :, :i_l] = wg[:, i0:i0 + i_l]
                gu[e, :, i_l:] = wu[:, i0:i0 + i_l]
                dn[e] = wd[i0:i0 + i_l]
            out[p + "gate_up_weight"] = gu
            out[p + "down_weight"] = dn
            if cfg.expert_bias:
                bgs, bds = nxt(), nxt()
                bgu = torch.empty((e_l, 2 * i_l), dtype=dtype, device=device)
                bd = torch.empty((e_l, H), dtype=dtype, device=device)
                for e in range(e_l):
                    ge = e0 + e
                    b = _normal((2 * I,), std, bgs * 1009 + ge, device, dtype)
                    bgu[e, :i_l] = b[i0:i0 + i_l]
                    bgu[e, i_l:] = b[I + i0:I + i0 + i_l]
                    b2 = _normal((H,), std, bds * 1009 + ge, device, dtype)
                    bd[e] = b2 if (moe_parallel == "ep" or rank == 0) else torch.zeros_like(b2)
                out[p + "gate_up_bias"] = bgu
                out[p + "down_bias"] = bd
    return out


def save_shard(weights: Dict[str, torch.Tensor], directory: str, rank: int) -> str:
    """Write ``shard_{rank}.safetensors`` (same file naming as the reference converter)."""
    from safetensors.torch import save_file

    os.makedirs(directory, exist_ok=True)
    path = os.path.join(directory, f"shard_{rank}.safetensors")
    save_file({k: v.contiguous().cpu() for k, v in weights.items()}, path)
    return path


def load_shard(directory: str, rank: int, device="cpu") -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return load_file(os.path.join(directory, f"shard_{rank}.safetensors"), device=str(device))


def to_device_layout(w: torch.Tensor) -> torch.Tensor:
    """``x @ W`` orientation [.., K, N] -> K-major [.., N, K] contiguous (the tcgen05 operand layout)."""
    return w.transpose(-1, -2).contiguous()
