"""Plain PyTorch implementation of the same decoder (no paging, no fusion): the
oracle of the model tests and the "PyTorch eager" baseline arm of the benchmarks.

It consumes the same per-rank weight dictionaries (``x @ W`` orientation) and,
with a process group, performs the tensor-parallel all-reduces / gathers through
``torch.distributed`` (NCCL + cuBLAS + SDPA on GPU) — the baseline the fused
sm_100a path is measured against.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..parallel.comm import TPGroup
from .config import ModelConfig, yarn_inv_freq
from .weights import kv_heads_for_rank


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


class EagerTransformer:
    """Dense-cache eager decoder.  `dtype` float32 gives the numerical oracle, bfloat16 the
    timed baseline."""

    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], tp: Optional[TPGroup] = None,
                 device="cpu", dtype=torch.float32, moe_parallel: str = "ep"):
        self.cfg, self.tp = cfg, tp or TPGroup.single()
        self.device, self.dtype = torch.device(device), dtype
        self.w = {k: (v.to(self.device).to(dtype) if v.dtype != torch.float32 or k.endswith("sinks")
                      else v.to(self.device)) for k, v in weights.items()}
        world, rank = self.tp.world_size, self.tp.rank
        self.nq = cfg.num_heads // world
        _, self.nkv = kv_heads_for_rank(cfg, rank, world)
        self.moe_parallel = moe_parallel
        inv_freq, scale = yarn_inv_freq(cfg)
        ang = torch.arange(cfg.max_position, dtype=torch.float64)[:, None] * inv_freq[None, :]
        self.cos = (ang.cos() * scale).float().to(self.device)
        self.sin = (ang.sin() * scale).float().to(self.device)
        self.k_cache: List[Optional[torch.Tensor]] = [None] * cfg.num_layers
        self.v_cache: List[Optional[torch.Tensor]] = [None] * cfg.num_layers

    def reset(self):
        self.k_cache = [None] * self.cfg.num_layers
        self.v_cache = [None] * self.cfg.num_layers

    def _rope(self, t, pos):
        d2 = self.cfg.head_dim // 2
        c, s = self.cos[pos][:, :, None, :], self.sin[pos][:, :, None, :]
        a, b = t[..., :d2].float(), t[..., d2:].float()
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(t.dtype)

    def _moe(self, p, x):
        cfg, w = self.cfg, self.w
        T, H = x.shape
        logits = x.float() @ w[p + "router_weight"].float()
        if cfg.router_bias:
            logits = logits + w[p + "router_bias"].float()
        if cfg.router_mode == "softmax_topk":
            pr = torch.softmax(logits, -1)
            wt, ex = pr.topk(cfg.top_k, -1)
            wt = wt / wt.sum(-1, keepdim=True)
        else:
            v, ex = logits.topk(cfg.top_k, -1)
            wt = torch.softmax(v, -1)
        gu, dn = w[p + "gate_up_weight"], w[p + "down_weight"]
        e_l = gu.shape[0]
        e0 = self.tp.rank * e_l if (self.moe_parallel == "ep" and self.tp.world_size > 1) else 0
        i_l = gu.shape[-1] // 2
        out = torch.zeros((T, H), dtype=torch.float32, device=x.device)
        for e in range(e_l):
            sel = (ex == e + e0)
            rows = sel.any(-1).nonzero().squeeze(-1)
            if rows.numel() == 0:
                continue
            xe = x[rows]
            h = xe @ gu[e]
            if cfg.expert_bias:
                h = h + w[p + "gate_up_bias"][e]
            g, u = h[:, :i_l].float(), h[:, i_l:].float()
            if cfg.swiglu_limit > 0:
                g = g.clamp(max=cfg.swiglu_limit)
                u = u.clamp(-cfg.swiglu_limit, cfg.swiglu_limit)
                a = (u + 1) * g * torch.sigmoid(cfg.swiglu_alpha * g)
            else:
                a = F.silu(g) * u
            y = a.to(x.dtype) @ dn[e]
            if cfg.expert_bias:
                y = y + w[p + "down_bias"][e]
            wsel = (wt * sel)[rows].sum(-1, keepdim=True)
            out[rows] += wsel * y.float()
        out = out.to(x.dtype)
        self.tp.all_reduce(out)
        return out

    def forward(self, ids: torch.Tensor, start_pos: int = 0, return_hidden: bool = False):
        """ids [B, S] -> final-normed hidden [B, S, H]; appends to the dense cache."""
        cfg, w = self.cfg, self.w
        B, S = ids.shape
        d = cfg.head_dim
        x = w["tok_embedding"][ids.long()]
        pos = torch.arange(start_pos, start_pos + S, device=self.device)[None, :].expand(B, S)
        taps = []
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            in_name = p + ("input_layernorm_weight" if p + "input_layernorm_weight" in w else "input_weight")
            post_name = p + ("post_attention_layernorm_weight" if p + "post_attention_layernorm_weight" in w
                             else "post_attention_weight")
            h = _rms(x, w[in_name], cfg.rms_eps)
            qkv = h @ w[p + "qkv_weight"]
            if cfg.attn_bias:
                qkv = qkv + w[p + "qkv_bias"]
            q, k, v = qkv.split([self.nq * d, self.nkv * d, self.nkv * d], dim=-1)
            q, k, v = q.reshape(B, S, self.nq, d), k.reshape(B, S, self.nkv, d), v.reshape(B, S, self.nkv, d)
            if cfg.qk_norm:
                q, k = _rms(q, w[p + "q_norm_weight"], cfg.rms_eps), _rms(k, w[p + "k_norm_weight"], cfg.rms_eps)
            q, k = self._rope(q, pos), self._rope(k, pos)
            if self.k_cache[i] is not None:
                k = torch.cat([self.k_cache[i], k], dim=1)
                v = torch.cat([self.v_cache[i], v], dim=1)
            self.k_cache[i], self.v_cache[i] = k, v
            L = k.shape[1]
            g = self.nq // self.nkv
            kk, vv = k.repeat_interleave(g, dim=2), v.repeat_interleave(g, dim=2)
            s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kk.float()) / math.sqrt(d)
            qp = pos[0][:, None]
            kp = torch.arange(L, device=self.device)[None, :]
            mask = torch.ones((S, L), dtype=torch.bool, device=self.device)
            if cfg.causal:
                mask &= kp <= qp
            win = cfg.window_for_layer(i)
            if win > 0:
                mask &= kp > qp - win
            s = s.masked_fill(~mask[None, None], float("-inf"))
            if cfg.attention_sinks:
                sk = w[p + "sinks"].float()[None, :, None, None].expand(B, self.nq, S, 1)
                pr = torch.softmax(torch.cat([s, sk], -1), -1)[..., :-1]
            else:
                pr = torch.softmax(s, -1)
            a = torch.einsum("bhqk,bkhd->bqhd", pr, vv.float()).to(x.dtype).reshape(B, S, self.nq * d)
            o = a @ w[p + "o_weight"]
            if cfg.attn_bias:
                o = o + w[p + "o_bias"]
            self.tp.all_reduce(o)
            x = x + o
            h = _rms(x, w[post_name], cfg.rms_eps)
            if cfg.is_moe:
                y = self._moe(p, h.reshape(B * S, -1)).reshape(B, S, -1)
            else:
                gu = h @ w[p + "gate_up_weight"]
                i_l = gu.shape[-1] // 2
                gg, uu = gu[..., :i_l].float(), gu[..., i_l:].float()
                if cfg.swiglu_limit > 0:
                    gg = gg.clamp(max=cfg.swiglu_limit)
                    uu = uu.clamp(-cfg.swiglu_limit, cfg.swiglu_limit)
                    act = (uu + 1) * gg * torch.sigmoid(cfg.swiglu_alpha * gg)
                else:
                    act = F.silu(gg) * uu
                y = act.to(x.dtype) @ w[p + "down_weight"]
                self.tp.all_reduce(y)
            x = x + y
            taps.append(x)
        out = _rms(x, w["norm_weight"], cfg.rms_eps)
        return (out, taps) if return_hidden else out

    # ------------------------------------------------------------------ timed baseline path
    def alloc_static_cache(self, batch: int, max_len: int) -> None:
        """Preallocated dense KV cache [B, kv_heads, max_len, d] per layer for `forward_sdpa`."""
        shape = (batch, self.nkv, max_len, self.cfg.head_dim)
        self.k_static = [torch.empty(shape, dtype=self.dtype, device=self.device) for _ in range(self.cfg.num_layers)]
        self.v_static = [torch.empty(shape, dtype=self.dtype, device=self.device) for _ in range(self.cfg.num_layers)]

    def forward_sdpa(self, ids: torch.Tensor, start_pos: int = 0) -> torch.Tensor:
        """The same decoder the way a PyTorch user would write it for speed: bf16 matmuls (cuBLAS),
        `scaled_dot_product_attention` with grouped-query heads over a preallocated dense cache, NCCL
        all-reduces.  Causal models without sliding windows or attention sinks only (Llama, Qwen3)."""
        cfg, w = self.cfg, self.w
        if cfg.attention_sinks or any(cfg.window_for_layer(i) > 0 for i in range(cfg.num_layers)):
            return self.forward(ids, start_pos)
        B, S = ids.shape
        d = cfg.head_dim
        x = w["tok_embedding"][ids.long()]
        pos = torch.arange(start_pos, start_pos + S, device=self.device)[None, :].expand(B, S)
        end = start_pos + S
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            in_name = p + ("input_layernorm_weight" if p + "input_layernorm_weight" in w else "input_weight")
            post_name = p + ("post_attention_layernorm_weight" if p + "post_attention_layernorm_weight" in w
                             else "post_attention_weight")
            h = _rms(x, w[in_name], cfg.rms_eps)
            qkv = h @ w[p + "qkv_weight"]
            if cfg.attn_bias:
                qkv = qkv + w[p + "qkv_bias"]
            q, k, v = qkv.split([self.nq * d, self.nkv * d, self.nkv * d], dim=-1)
            q, k, v = q.reshape(B, S, self.nq, d), k.reshape(B, S, self.nkv, d), v.reshape(B, S, self.nkv, d)
            if cfg.qk_norm:
                q, k = _rms(q, w[p + "q_norm_weight"], cfg.rms_eps), _rms(k, w[p + "k_norm_weight"], cfg.rms_eps)
            q, k = self._rope(q, pos), self._rope(k, pos)
            self.k_static[i][:, :, start_pos:end] = k.transpose(1, 2)
            self.v_static[i][:, :, start_pos:end] = v.transpose(1, 2)
            if S == 1:
                # decode: the g query heads of a kv head act as g query rows, so the fused attention
                # kernels apply without materialising repeated K / V
                g = self.nq // self.nkv
                a = F.scaled_dot_product_attention(q.reshape(B, self.nkv, g, d), self.k_static[i][:, :, :end],
                                                   self.v_static[i][:, :, :end])
                a = a.reshape(B, 1, self.nq * d)
            else:
                a = F.scaled_dot_product_attention(q.transpose(1, 2), self.k_static[i][:, :, :end],
                                                   self.v_static[i][:, :, :end],
                                                   is_causal=(S > 1 and start_pos == 0), enable_gqa=True)
                a = a.transpose(1, 2).reshape(B, S, self.nq * d)
            o = a @ w[p + "o_weight"]
            if cfg.attn_bias:
                o = o + w[p + "o_bias"]
            self.tp.all_reduce(o)
            x = x + o
            h = _rms(x, w[post_name], cfg.rms_eps)
            if cfg.is_moe:
                y = self._moe(p, h.reshape(B * S, -1)).reshape(B, S, -1)
            else:
                gu = h @ w[p + "gate_up_weight"]
                i_l = gu.shape[-1] // 2
                y = (F.silu(gu[..., :i_l]) * gu[..., i_l:]) @ w[p + "down_weight"]
                self.tp.all_reduce(y)
            x = x + y
        return _rms(x, w["norm_weight"], cfg.rms_eps)

    def forward_decode_static(self, ids: torch.Tensor, pos_t: torch.Tensor) -> torch.Tensor:
        """One decode step whose position is a device tensor (int64 [1]), so the step can be captured in a CUDA
        graph and replayed: the cache row is written with `index_copy_`, attention runs over the whole static
        cache under a mask `key position <= pos`.  Dense-FFN causal models only (the expert loops of the MoE
        path branch on device data)."""
        cfg, w = self.cfg, self.w
        if cfg.is_moe or cfg.attention_sinks or any(cfg.window_for_layer(i) > 0 for i in range(cfg.num_layers)):
            raise NotImplementedError("graph-capturable eager decode covers dense causal models")
        B = ids.shape[0]
        d = cfg.head_dim
        max_len = self.k_static[0].shape[2]
        x = w["tok_embedding"][ids.long()]
        pos = pos_t[None, :].expand(B, 1)
        mask = (torch.arange(max_len, device=self.device) <= pos_t)[None, None, None, :]
        g = self.nq // self.nkv
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            in_name = p + ("input_layernorm_weight" if p + "input_layernorm_weight" in w else "input_weight")
            post_name = p + ("post_attention_layernorm_weight" if p + "post_attention_layernorm_weight" in w
                             else "post_attention_weight")
            h = _rms(x, w[in_name], cfg.rms_eps)
            qkv = h @ w[p + "qkv_weight"]
            if cfg.attn_bias:
                qkv = qkv + w[p + "qkv_bias"]
            q, k, v = qkv.split([self.nq * d, self.nkv * d, self.nkv * d], dim=-1)
            q, k, v = q.reshape(B, 1, self.nq, d), k.reshape(B, 1, self.nkv, d), v.reshape(B, 1, self.nkv, d)
            if cfg.qk_norm:
                q, k = _rms(q, w[p + "q_norm_weight"], cfg.rms_eps), _rms(k, w[p + "k_norm_weight"], cfg.rms_eps)
            q, k = self._rope(q, pos), self._rope(k, pos)
            self.k_static[i].index_copy_(2, pos_t, k.transpose(1, 2))
            self.v_static[i].index_copy_(2, pos_t, v.transpose(1, 2))
            a = F.scaled_dot_product_attention(q.reshape(B, self.nkv, g, d), self.k_static[i], self.v_static[i],
                                               attn_mask=mask)
            o = a.reshape(B, 1, self.nq * d) @ w[p + "o_weight"]
            if cfg.attn_bias:
                o = o + w[p + "o_bias"]
            self.tp.all_reduce(o)
            x = x + o
            h = _rms(x, w[post_name], cfg.rms_eps)
            gu = h @ w[p + "gate_up_weight"]
            i_l = gu.shape[-1] // 2
            y = (F.silu(gu[..., :i_l]) * gu[..., i_l:]) @ w[p + "down_weight"]
            self.tp.all_reduce(y)
            x = x + y
        return _rms(x, w["norm_weight"], cfg.rms_eps)

    def greedy(self, hidden_last: torch.Tensor) -> torch.Tensor:
        """hidden_last [B, H] -> global greedy ids (vocab-parallel aware)."""
        logits = (hidden_last @ self.w["lm_head_weight"]).float()
        vals, ids = logits.max(-1)
        if self.tp.world_size == 1:
            return ids.to(torch.int32)
        ids = ids + self.tp.rank * logits.shape[-1]
        allp = self.tp.all_gather(torch.stack([vals, ids.float()], -1))
        best = allp[..., 0].argmax(0)
        return allp[..., 1].gather(0, best[None]).squeeze(0).to(torch.int32)

    def generate(self, prompts: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        """prompts [B, S] (equal lengths) -> new tokens [B, max_new_tokens]."""
        self.reset()
        h = self.forward(prompts, 0)
        nxt = self.greedy(h[:, -1])
        outs = [nxt]
        pos = prompts.shape[1]
        for _ in range(max_new_tokens - 1):
            h = self.forward(nxt[:, None], pos)
            nxt = self.greedy(h[:, -1])
            outs.append(nxt)
            pos += 1
        return torch.stack(outs, dim=1)
