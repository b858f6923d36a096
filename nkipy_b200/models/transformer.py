"""Decoder-only transformer on the hand-written sm_100a operators.

The forward pass is the reference's layer structure — RMSNorm -> fused QKV ->
(QK-norm) -> RoPE -> KV-cache write -> attention -> o_proj -> all-reduce ->
residual -> RMSNorm -> FFN / MoE -> all-reduce -> residual
(examples/models/qwen3/kernels/transformer_layer.py:16-120,
examples/models/qwen3/kernels/attention.py:25-156) — but organised around what a
B200 wants: a paged KV cache, one packed token batch per prefill, and a decode
step made of a handful of fused launches per layer that is captured in a CUDA
graph:

    decode layer (tp = 1):  qkv GEMM (split-K partials) -> [sum + RoPE + cache append]
        -> paged attention -> o GEMM (split-K) -> [sum + residual + RMSNorm]
        -> gate_up GEMM with SwiGLU epilogue -> down GEMM (split-K) -> [sum + residual + RMSNorm]

Tensor parallelism follows the reference (column-parallel qkv / gate_up / lm_head,
row-parallel o / down, two reductions per layer, vocab-parallel argmax gathered
over ranks, examples/models/qwen3/kernels/sampling.py:127-147).
"""

from __future__ import annotations

import math
import os
from typing import Dict, List, Optional

import torch

from .. import ops
from ..parallel.comm import TPGroup
from .config import ModelConfig, yarn_inv_freq
from .kv_cache import PagedKVCache
from .weights import kv_heads_for_rank, to_device_layout


def pick_splits(n_out: int, k: int, sms: int = 148) -> int:
    """Split-K factor for a decode-sized GEMM.  Two CTAs share an SM in that orientation,
    so aim for about two CTAs per SM while each split still streams at least 512
    contraction elements."""
    tiles = (n_out + 127) // 128
    if tiles >= 2 * sms * 3 // 4:
        return 1
    want = max(1, (2 * sms) // tiles)
    min_k = int(os.environ.get("NKIPY_B200_SPLIT_MIN_K", "512"))
    return max(1, min(want, k // min_k, 8))


def pick_cluster_splits(tiles: int, k: int, tokens: int, sms: int = 148) -> int:
    """Cluster size (= split-K factor: 1, 2, 4 or 8) of the decode GEMM whose split-K sum happens inside the
    kernel (`ops.decode_linear`): double it while the grid still fits the resident CTA slots (two CTAs per SM
    up to 64 tokens, one above) and every split keeps at least two 64-wide k-blocks."""
    slots = sms * (2 if tokens <= 64 else 1)
    kb = max(1, k // 64)
    s = 1
    while s < 8 and tiles * s * 2 <= slots and kb // (s * 2) >= 2:
        s *= 2
    return s


class LayerWeights:
    __slots__ = ("qkv", "o", "gate_up", "down", "input_norm", "post_norm", "q_norm", "k_norm", "qkv_bias", "o_bias",
                 "sinks", "router", "router_bias", "gate_up_bias", "down_bias")

    def __init__(self):
        for s in self.__slots__:
            setattr(self, s, None)


class TransformerLM:
    """Weights + forward passes of one tensor-parallel rank."""

    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], tp: Optional[TPGroup] = None,
                 device=None, moe_parallel: str = "ep", force_fused: bool = False):
        self.cfg = cfg
        # force_fused: take the peer-memory (push + reduce) kernels even with one rank, whose only peer is
        # then this GPU itself (single-GPU profiles of the multi-GPU decode path)
        self.force_fused = force_fused
        self.tp = tp or TPGroup.single()
        self.device = torch.device(device if device is not None else weights["tok_embedding"].device)
        world, rank = self.tp.world_size, self.tp.rank
        self.nq = cfg.num_heads // world
        self.kv0, self.nkv = kv_heads_for_rank(cfg, rank, world)
        self.d = cfg.head_dim
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        self.moe_parallel = moe_parallel
        dev = self.device

        def get(name):
            return weights[name].to(dev)

        self.tok_embedding = get("tok_embedding").contiguous()
        self.final_norm = get("norm_weight")
        self.lm_head = to_device_layout(get("lm_head_weight"))        # [V/tp, H]
        self.vocab_local = self.lm_head.shape[0]
        self.layers: List[LayerWeights] = []
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            lw = LayerWeights()
            lw.qkv = to_device_layout(get(p + "qkv_weight"))
            lw.o = to_device_layout(get(p + "o_weight"))
            norm_in = p + ("input_layernorm_weight" if p + "input_layernorm_weight" in weights else "input_weight")
            norm_post = p + ("post_attention_layernorm_weight" if p + "post_attention_layernorm_weight" in weights
                             else "post_attention_weight")
            lw.input_norm = get(norm_in)
            lw.post_norm = get(norm_post)
            if cfg.qk_norm:
                lw.q_norm, lw.k_norm = get(p + "q_norm_weight"), get(p + "k_norm_weight")
            if cfg.attn_bias:
                lw.qkv_bias, lw.o_bias = get(p + "qkv_bias"), get(p + "o_bias")
            if cfg.attention_sinks:
                lw.sinks = get(p + "sinks").float().contiguous()
            if cfg.is_moe:
                lw.router = to_device_layout(get(p + "router_weight"))            # [E, H]
                lw.router_bias = get(p + "router_bias") if cfg.router_bias else None
                lw.gate_up = to_device_layout(get(p + "gate_up_weight"))          # [E_l, 2 I_l, H]
                lw.down = to_device_layout(get(p + "down_weight"))                # [E_l, H, I_l]
                if cfg.expert_bias:
                    lw.gate_up_bias, lw.down_bias = get(p + "gate_up_bias"), get(p + "down_bias")
            else:
                lw.gate_up = to_device_layout(get(p + "gate_up_weight"))          # [2 I_l, H]
                lw.down = to_device_layout(get(p + "down_weight"))                # [H, I_l]
            self.layers.append(lw)
        inv_freq, rope_scale = yarn_inv_freq(cfg)
        self.rope = ops.rope_table(cfg.head_dim, cfg.max_position, inv_freq=inv_freq, scaling=rope_scale, device=dev)
        self._moe = None
        if cfg.is_moe:
            from .moe import MoEBlock

            self._moe = MoEBlock(cfg, self.tp, moe_parallel)
        # decode split-K factors (per GEMM shape)
        H = cfg.hidden_size
        self.split_qkv = pick_splits(self.layers[0].qkv.shape[0], H)
        self.split_o = pick_splits(H, self.layers[0].o.shape[1])
        self.split_down = 1 if cfg.is_moe else pick_splits(H, self.layers[0].down.shape[1])
        # "legacy": persistent split-K GEMMs that leave fp32 partials to the next kernel; otherwise the projections
        # finish their own split-K sum and apply RoPE / SwiGLU / the push themselves (ops.DECODE_GEMM_IMPL)
        self.cluster_gemm = ops.DECODE_GEMM_IMPL != "legacy"
        self.fix_gemm = ops.DECODE_GEMM_IMPL == "fixup"
        self.split_gate_up = 1
        if not cfg.is_moe:
            two_i = self.layers[0].gate_up.shape[0]
            if two_i // 256 < 100:          # fewer than ~100 fused gate/up tile pairs
                self.split_gate_up = max(2, pick_splits(two_i, H))

    # ------------------------------------------------------------------ cache
    def new_cache(self, num_blocks: int, max_batch: int, max_seq_len: int,
                  enable_prefix_sharing: bool = True) -> PagedKVCache:
        max_blocks = (max_seq_len + self.cfg.block_size - 1) // self.cfg.block_size
        return PagedKVCache(self.cfg.num_layers, self.nkv, self.d, num_blocks, max_batch, max_blocks, self.device,
                            enable_prefix_sharing=enable_prefix_sharing)

    def weight_bytes(self) -> int:
        n = self.tok_embedding.numel() + self.lm_head.numel()
        for lw in self.layers:
            for s in ("qkv", "o", "gate_up", "down", "router"):
                t = getattr(lw, s)
                if t is not None:
                    n += t.numel()
        return n * 2

    # ------------------------------------------------------------------ FFN
    def _csplits(self, w: torch.Tensor, tokens: int, gated: bool = False) -> int:
        """Cluster split factor for a decode GEMM with this weight and token count (cached per shape)."""
        key = (w.shape[0], w.shape[1], tokens, gated)
        cache = self.__dict__.setdefault("_csplit_cache", {})
        if key not in cache:
            if self.fix_gemm:
                cache[key] = pick_splits(w.shape[0], w.shape[1])
            else:
                tiles = (w.shape[0] // 2 + 63) // 64 if gated else (w.shape[0] + 127) // 128
                cache[key] = pick_cluster_splits(tiles, w.shape[1], tokens)
        return cache[key]

    def _ffn_decode(self, lw: LayerWeights, normed: torch.Tensor, resid: torch.Tensor, next_norm: torch.Tensor):
        """Returns (new residual, normed for the next block)."""
        cfg = self.cfg
        if cfg.is_moe:
            return self._moe.forward_add_rmsnorm(lw, normed, resid, next_norm)
        T = normed.shape[0]
        if self.cluster_gemm and T <= 128 and normed.is_cuda:
            # gate / up with the split-K sum and SwiGLU inside one kernel
            act = ops.decode_linear(normed, lw.gate_up, gated=True, splits=self._csplits(lw.gate_up, T, True),
                                    act_limit=cfg.swiglu_limit, act_alpha=cfg.swiglu_alpha)
            return self._row_parallel_reduce(act, lw.down, self._csplits(lw.down, T), resid, next_norm, None)
        if cfg.swiglu_limit <= 0 and self.split_gate_up == 1:
            act = ops.linear(normed, lw.gate_up, gated=True)
        elif self.split_gate_up > 1:
            # too few gate/up tile pairs to fill the SMs: split-K partials, gate applied by the reducer
            act = ops.silu_mul(ops.linear(normed, lw.gate_up, splits=self.split_gate_up), limit=cfg.swiglu_limit,
                               alpha=cfg.swiglu_alpha)
        else:
            act = ops.silu_mul(ops.linear(normed, lw.gate_up), limit=cfg.swiglu_limit, alpha=cfg.swiglu_alpha)
        return self._row_parallel_reduce(act, lw.down, self.split_down, resid, next_norm, None)

    def _row_parallel_reduce(self, x, w, splits, resid, next_norm, bias):
        """Row-parallel GEMM + sum over ranks + residual + next RMSNorm (decode-sized M)."""
        cfg = self.cfg
        if self.tp.world_size == 1 and not (self.force_fused and getattr(self.tp, "fused", None) is not None):
            if self.cluster_gemm and x.shape[0] <= 128 and x.is_cuda:
                h = ops.decode_linear(x, w, splits=splits, bias=bias, residual=resid)
                return h, ops.rmsnorm(h, next_norm, cfg.rms_eps)
            if splits > 1:
                parts = ops.linear(x, w, splits=splits)
                return ops.add_rmsnorm(None, next_norm, residual_in=resid, partials=parts, bias=bias,
                                       eps=cfg.rms_eps)
            y = ops.linear(x, w)
            return ops.add_rmsnorm(y, next_norm, residual_in=resid, bias=bias, eps=cfg.rms_eps)
        fused = getattr(self.tp, "fused", None)
        if fused is not None:
            return fused.gemm_allreduce_add_rmsnorm(x, w, resid, next_norm, bias, cfg.rms_eps, splits)
        if splits > 1:
            y = ops.reduce_partials(ops.linear(x, w, splits=splits))
        else:
            y = ops.linear(x, w)
        self.tp.all_reduce(y)
        return ops.add_rmsnorm(y, next_norm, residual_in=resid, bias=bias, eps=cfg.rms_eps)

    # ------------------------------------------------------------------ decode
    def decode_step(self, ids: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, cache: PagedKVCache,
                    block_table: torch.Tensor, context_lens: torch.Tensor, q_len: int = 1,
                    return_hidden: bool = False, inputs=None) -> torch.Tensor:
        """One decode (or q_len-token verify) step for the batch.  ids [B * q_len] int32;
        context_lens already count the new tokens.  Returns the final-normed hidden
        states [B * q_len, H] (with return_hidden also the residual stream after every layer).
        inputs = (residual [T, H], first-layer input [T, K0]) replaces the embedding lookup and the
        first norm (used by models whose first layer consumes something else than token embeddings)."""
        cfg = self.cfg
        if inputs is None:
            x = ops.embedding(ids, self.tok_embedding)
            resid = x
            normed = ops.rmsnorm(x, self.layers[0].input_norm, cfg.rms_eps)
        else:
            resid, normed = inputs
        taps = [] if return_hidden else None
        T = normed.shape[0]
        if self._persistent_layers(T, normed):
            return self._decode_step_persistent(resid, normed, positions, slots, cache, block_table, context_lens,
                                                q_len, taps)
        cluster = self.cluster_gemm and T <= 128 and normed.is_cuda and self.d in (64, 128)
        for i, lw in enumerate(self.layers):
            if cluster:
                # QKV projection, QK-norm, RoPE and the cache append in one launch
                q = ops.qkv_rope_append(normed, lw.qkv, positions, slots, self.rope, cache.k[i], cache.v[i], self.nq,
                                        self.nkv, self.d, splits=self._csplits(lw.qkv, T), bias=lw.qkv_bias,
                                        q_norm_w=lw.q_norm, k_norm_w=lw.k_norm, norm_eps=cfg.rms_eps)
            else:
                if self.split_qkv > 1:
                    qkv = ops.linear(normed, lw.qkv, splits=self.split_qkv)
                else:
                    qkv = ops.linear(normed, lw.qkv)
                if (ops.fused_rope_attn_enabled(self.tp.world_size) and q_len == 1 and qkv.dtype == torch.float32 and qkv.is_cuda
                        and self.d in (64, 128) and self.nq // self.nkv <= 16):
                    # RoPE and the cache append run inside the attention kernel: one launch less per layer
                    q = None
                    attn = ops.rope_attn_decode(qkv, positions, slots, self.rope, cache.k[i], cache.v[i], block_table,
                                                context_lens, self.scale, self.nq, self.nkv, bias=lw.qkv_bias,
                                                q_norm_w=lw.q_norm, k_norm_w=lw.k_norm, norm_eps=cfg.rms_eps,
                                                window=cfg.window_for_layer(i), sinks=lw.sinks)
                else:
                    q = ops.rope_kv_append(qkv, positions, slots, self.rope, cache.k[i], cache.v[i], self.nq,
                                           self.nkv, self.d, bias=lw.qkv_bias, q_norm_w=lw.q_norm,
                                           k_norm_w=lw.k_norm, norm_eps=cfg.rms_eps)
            if q is not None:
                attn = ops.paged_attn_decode(q, cache.k[i], cache.v[i], block_table, context_lens, self.scale,
                                             q_len=q_len, window=cfg.window_for_layer(i), sinks=lw.sinks)
            split_o = self._csplits(lw.o, T) if cluster else self.split_o
            resid, normed = self._row_parallel_reduce(attn, lw.o, split_o, resid, lw.post_norm, lw.o_bias)
            nxt = self.layers[i + 1].input_norm if i + 1 < len(self.layers) else self.final_norm
            resid, normed = self._ffn_decode(lw, normed, resid, nxt)
            if taps is not None:
                taps.append(resid)
        if return_hidden:
            return normed, taps
        return normed

    # ------------------------------------------------------------------ decode, one launch per layer
    def _persistent_layers(self, T: int, normed: torch.Tensor) -> bool:
        """Whether the decode step runs on the persistent layer kernel: dense-FFN models on a GPU, at most 128
        tokens, and either one rank or the fused tensor-parallel buffers."""
        if ops.DECODE_LAYER_IMPL != "persistent" or not normed.is_cuda or T > 128:
            return False
        if self.d not in (64, 128, 256) or self.cfg.hidden_size % 8 or self.cfg.hidden_size > 6144:
            return False
        if self.tp.world_size > 1 or self.force_fused:
            fused = getattr(self.tp, "fused", None)
            return fused is not None and T <= fused.max_tokens
        return True

    def _layer_splits(self):
        """Split-K factors (o, gate/up, down, qkv) of the persistent layer kernel's GEMM stages, and whether
        gate / up applies SwiGLU in its own epilogue (enough tile pairs to fill the SMs) or from partials."""
        if getattr(self, "_lsplits", None) is None:
            from ..ops.decode_layer import env_splits, pick_layer_splits

            lw, H = self.layers[0], self.cfg.hidden_size
            if self.cfg.is_moe:              # the experts run in their own kernels: only the two ends are stages
                inter, fused_gate = 0, False
                s = [pick_layer_splits(H, lw.o.shape[1]), 1, 1, pick_layer_splits(lw.qkv.shape[0], H)]
            else:
                inter = lw.gate_up.shape[0] // 2
                fused_gate = self.cfg.swiglu_limit <= 0 and lw.gate_up_bias is None and inter // 128 >= 100
                s = [pick_layer_splits(H, lw.o.shape[1]), 1 if fused_gate else pick_layer_splits(2 * inter, H),
                     pick_layer_splits(H, lw.down.shape[1]), pick_layer_splits(lw.qkv.shape[0], H)]
            env = env_splits()
            if env:
                s = [e if e > 0 else d for e, d in zip(env, s)]
                if env[1] > 1:
                    fused_gate = False
            fused = getattr(self.tp, "fused", None)
            if fused is not None and (self.tp.world_size > 1 or self.force_fused):
                s[0], s[2] = min(s[0], fused.max_splits), min(s[2], fused.max_splits)
            self._lsplits = (tuple(s), fused_gate)
        return self._lsplits

    def _decode_step_persistent(self, resid, normed, positions, slots, cache, block_table, context_lens, q_len, taps):
        """The decode step as  QKV+RoPE(layer 0), then per layer: attention, one persistent launch."""
        from ..ops import decode_layer as DL

        cfg = self.cfg
        T, H = normed.shape
        dev = normed.device
        (s_o, s_gu, s_down, s_qkv), fused_gate = self._layer_splits()
        lw0 = self.layers[0]
        moe = cfg.is_moe
        inter = 0 if moe else lw0.gate_up.shape[0] // 2
        qkv_w = lw0.qkv.shape[0]
        scratch = DL.layer_scratch(dev, DL.scratch_floats(DL.block_n_for(T), [
            (H, s_o), (0 if fused_gate else 2 * inter, s_gu), (H, s_down), (qkv_w, s_qkv)]))
        fused = getattr(self.tp, "fused", None) if (self.tp.world_size > 1 or self.force_fused) else None
        bf = dict(dtype=torch.bfloat16, device=dev)

        def qkv_args(i, q_out):
            lw = self.layers[i]
            return dict(w_qkv=lw.qkv, splits_qkv=s_qkv, nq=self.nq, nkv=self.nkv, head_dim=self.d, bias_qkv=lw.qkv_bias,
                        positions=positions, slots=slots, cos_sin=self.rope, q_norm_w=lw.q_norm, k_norm_w=lw.k_norm,
                        q_out=q_out, k_cache=cache.k[i], v_cache=cache.v[i])

        q = torch.empty((T, self.nq * self.d), **bf)
        DL.decode_layer(DL.ST_QKV | DL.ST_ROPE, T, H, cfg.rms_eps, scratch, normed_out=normed, **qkv_args(0, q))
        n_layers = len(self.layers)
        for i, lw in enumerate(self.layers):
            attn = ops.paged_attn_decode(q, cache.k[i], cache.v[i], block_table, context_lens, self.scale,
                                         q_len=q_len, window=cfg.window_for_layer(i), sinks=lw.sinks)
            last = i + 1 == n_layers
            if moe:
                q, resid, normed = self._moe_layer_persistent(DL, i, lw, attn, resid, scratch, fused, qkv_args, T, H,
                                                              s_o, last)
                if taps is not None:
                    taps.append(resid)
                continue
            mask = DL.ST_O | DL.ST_RED1 | DL.ST_GU | DL.ST_DOWN | DL.ST_RED2
            if not fused_gate:
                mask |= DL.ST_SILU
            resid_mid, normed_mid = torch.empty((T, H), **bf), torch.empty((T, H), **bf)
            resid_out, normed_out = torch.empty((T, H), **bf), torch.empty((T, H), **bf)
            act = torch.empty((T, inter), **bf)
            extra = {}
            if not last:
                mask |= DL.ST_QKV | DL.ST_ROPE
                q = torch.empty((T, self.nq * self.d), **bf)
                extra = qkv_args(i + 1, q)
            DL.decode_layer(mask, T, H, cfg.rms_eps, scratch,
                            w_o=lw.o, attn=attn, splits_o=s_o, bias_o=lw.o_bias,
                            resid_in=resid, norm1_w=lw.post_norm, resid_mid=resid_mid, normed_mid=normed_mid,
                            w_gu=lw.gate_up, inter=inter, splits_gu=s_gu, fused_gate=fused_gate,
                            bias_gu=lw.gate_up_bias, act_limit=cfg.swiglu_limit, act_alpha=cfg.swiglu_alpha, act=act,
                            w_down=lw.down, splits_down=s_down, bias_down=lw.down_bias,
                            norm2_w=self.final_norm if last else self.layers[i + 1].input_norm,
                            resid_out=resid_out, normed_out=normed_out,
                            tp_buffers=None if fused is None else fused.layer_buffers(T, H), **extra)
            resid, normed = resid_out, normed_out
            if taps is not None:
                taps.append(resid)
        if taps is not None:
            return normed, taps
        return normed

    def _moe_layer_persistent(self, DL, i, lw, attn, resid, scratch, fused, qkv_args, T, H, s_o, last):
        """A mixture-of-experts layer around the persistent kernel: launch A runs o_proj and the first reduction,
        the experts run in their own kernels, launch B sums their outputs (pushed by every rank, or local),
        adds the residual, norms, and runs the next layer's QKV projection with RoPE and the cache append."""
        cfg = self.cfg
        bf = dict(dtype=torch.bfloat16, device=attn.device)
        resid_mid, normed_mid = torch.empty((T, H), **bf), torch.empty((T, H), **bf)
        buf_o = None if fused is None else fused.next_buffer(T, H)
        DL.decode_layer(DL.ST_O | DL.ST_RED1, T, H, cfg.rms_eps, scratch, w_o=lw.o, attn=attn, splits_o=s_o,
                        bias_o=lw.o_bias, resid_in=resid, norm1_w=lw.post_norm, resid_mid=resid_mid,
                        normed_mid=normed_mid, tp_buffers=None if buf_o is None else (buf_o, buf_o))
        resid_out, normed_out = torch.empty((T, H), **bf), torch.empty((T, H), **bf)
        mask, extra, q = DL.ST_RED2, {}, None
        if not last:
            mask |= DL.ST_QKV | DL.ST_ROPE
            q = torch.empty((T, self.nq * self.d), **bf)
            extra = qkv_args(i + 1, q)
        norm2 = self.final_norm if last else self.layers[i + 1].input_norm
        if fused is not None:
            y_sorted, plan, weights = self._moe._experts(lw, normed_mid)
            b = fused.moe_combine_push(y_sorted, plan.pair_pos, weights, T)
            buf = fused.buffer(b)
            DL.decode_layer(mask, T, H, cfg.rms_eps, scratch, resid_mid=resid_mid, norm2_w=norm2, resid_out=resid_out,
                            normed_out=normed_out, tp_buffers=(buf, buf), red2_slots=self.tp.world_size, **extra)
        else:
            y = self._moe.forward(lw, normed_mid)
            DL.decode_layer(mask, T, H, cfg.rms_eps, scratch, resid_mid=resid_mid, norm2_w=norm2, resid_out=resid_out,
                            normed_out=normed_out, red2_x=y, **extra)
        return q, resid_out, normed_out

    # ------------------------------------------------------------------ prefill
    def prefill(self, ids: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, cache: PagedKVCache,
                block_table: torch.Tensor, q_start: torch.Tensor, q_lens: torch.Tensor, context_lens: torch.Tensor,
                max_q_len: int, return_hidden: bool = False, inputs=None):
        """Packed prefill of several sequences.  ids / positions / slots [T]; returns the
        final-normed hidden states [T, H] (and the per-layer residual streams when
        return_hidden is set, for speculative-decoding taps).  inputs: see `decode_step`."""
        cfg = self.cfg
        tp1 = self.tp.world_size == 1
        if (not tp1 and not return_hidden and inputs is None and getattr(self.tp, "fused", None) is not None
                and ids.shape[0] % self.tp.world_size == 0 and ids.shape[0] >= 128 * self.tp.world_size
                and ids.shape[0] <= self._sp_max_rows()):
            return self._prefill_sequence_parallel(ids, positions, slots, cache, block_table, q_start, q_lens,
                                                   context_lens, max_q_len)
        if inputs is None:
            x = ops.embedding(ids, self.tok_embedding)
            resid = x
            normed = ops.rmsnorm(x, self.layers[0].input_norm, cfg.rms_eps)
        else:
            resid, normed = inputs
        taps = [] if return_hidden else None
        for i, lw in enumerate(self.layers):
            qkv = ops.linear(normed, lw.qkv, swap=False)
            q = ops.rope_kv_append(qkv, positions, slots, self.rope, cache.k[i], cache.v[i], self.nq, self.nkv,
                                   self.d, bias=lw.qkv_bias, q_norm_w=lw.q_norm, k_norm_w=lw.k_norm,
                                   norm_eps=cfg.rms_eps)
            attn = ops.flash_attn_prefill(q, cache.k[i], cache.v[i], block_table, q_start, q_lens, context_lens,
                                          self.scale, max_q_len=max_q_len, causal=cfg.causal,
                                          window=cfg.window_for_layer(i), sinks=lw.sinks)
            if tp1:
                resid = ops.linear(attn, lw.o, swap=False, residual=resid, bias=lw.o_bias)
                normed = ops.rmsnorm(resid, lw.post_norm, cfg.rms_eps)
            else:
                o = ops.linear(attn, lw.o, swap=False, bias=lw.o_bias)
                self.tp.all_reduce(o)
                resid, normed = ops.add_rmsnorm(o, lw.post_norm, residual_in=resid, eps=cfg.rms_eps)
            nxt = self.layers[i + 1].input_norm if i + 1 < len(self.layers) else self.final_norm
            if cfg.is_moe:
                y = self._moe.forward(lw, normed)
                resid, normed = ops.add_rmsnorm(y, nxt, residual_in=resid, eps=cfg.rms_eps)
            else:
                if cfg.swiglu_limit <= 0:
                    act = ops.linear(normed, lw.gate_up, gated=True, swap=False)
                else:
                    act = ops.silu_mul(ops.linear(normed, lw.gate_up, swap=False), limit=cfg.swiglu_limit,
                                       alpha=cfg.swiglu_alpha)
                if tp1:
                    resid = ops.linear(act, lw.down, swap=False, residual=resid)
                    normed = ops.rmsnorm(resid, nxt, cfg.rms_eps)
                else:
                    dn = ops.linear(act, lw.down, swap=False)
                    self.tp.all_reduce(dn)
                    resid, normed = ops.add_rmsnorm(dn, nxt, residual_in=resid, eps=cfg.rms_eps)
            if taps is not None:
                taps.append(resid)
        if return_hidden:
            return normed, taps
        return normed

    SP_MIN_CAPACITY = 16384       # tokens; the engine's default prefill chunk
    # Local token count from which the MoE block of the sequence-parallel prefill exchanges tokens with the
    # expert owners (all-to-all in peer memory) instead of replicating them: below it the exchange's fixed
    # cost (count round trip, per-expert counters) outweighs the bytes saved.
    MOE_A2A_MIN_TOKENS = 256

    def _sp_max_rows(self) -> int:
        """Longest chunk the fused sequence-parallel kernels can describe; longer ones take the NCCL path."""
        from ..parallel.symm import _FusedGemmCollective

        return _FusedGemmCollective.max_rows(self.tp.world_size) // 2

    def _sp_pair(self, tokens: int):
        """The (reduce-scatter GEMM, all-gather GEMM) pair of the sequence-parallel prefill.  One pair serves
        every prompt length up to its capacity (the kernels take the row count per call); a longer chunk
        replaces it with one of twice the size, releasing the old symmetric buffers first, so the buffers
        neither multiply with the number of distinct prompt lengths nor are set up inside the hot path more
        than a handful of times."""
        from ..parallel.symm import AllGatherGemm, GemmReduceScatter

        pair = getattr(self, "_sp_ops", None)
        if pair is not None and tokens <= pair[0].m:
            return pair
        n = self.tp.world_size
        cap = max(self.SP_MIN_CAPACITY, pair[0].m if pair is not None else 0)
        while cap < tokens:
            cap *= 2
        cap = (cap + 128 * n - 1) // (128 * n) * (128 * n)
        if pair is not None:
            pair[0].close()
            pair[1].close()
        self._sp_ops = (GemmReduceScatter(self.tp, cap, self.cfg.hidden_size),
                        AllGatherGemm(self.tp, cap, self.cfg.hidden_size))
        return self._sp_ops

    def _prefill_sequence_parallel(self, ids, positions, slots, cache, block_table, q_start, q_lens, context_lens,
                                   max_q_len):
        """Prefill for tp > 1 in the sequence-parallel layout: the residual stream lives as one row slab
        [T / tp, H] per rank, the column-parallel projections gather the slabs inside the GEMM kernel
        (`AllGatherGemm`) and the row-parallel projections reduce-scatter inside theirs
        (`GemmReduceScatter`), so no library collective sits between the GEMMs of a layer."""
        from ..parallel.symm import AllGatherGemm, GemmReduceScatter

        cfg, tp = self.cfg, self.tp
        T = ids.shape[0]
        n, r = tp.world_size, tp.rank
        rows = T // n
        rs, ag = self._sp_pair(T)
        if not hasattr(self, "_o_bias_full"):
            # the row-parallel bias is stored on rank 0 only (zeros elsewhere); every slab needs it
            self._o_bias_full = [None if lw.o_bias is None else tp.all_reduce(lw.o_bias.clone())
                                 for lw in self.layers]
        resid = ops.embedding(ids[r * rows:(r + 1) * rows], self.tok_embedding)
        normed = ops.rmsnorm(resid, self.layers[0].input_norm, cfg.rms_eps)
        for i, lw in enumerate(self.layers):
            qkv = ag(normed, lw.qkv)
            q = ops.rope_kv_append(qkv, positions, slots, self.rope, cache.k[i], cache.v[i], self.nq, self.nkv,
                                   self.d, bias=lw.qkv_bias, q_norm_w=lw.q_norm, k_norm_w=lw.k_norm,
                                   norm_eps=cfg.rms_eps)
            attn = ops.flash_attn_prefill(q, cache.k[i], cache.v[i], block_table, q_start, q_lens, context_lens,
                                          self.scale, max_q_len=max_q_len, causal=cfg.causal,
                                          window=cfg.window_for_layer(i), sinks=lw.sinks)
            o = rs(attn, lw.o)
            resid, normed = ops.add_rmsnorm(o, lw.post_norm, residual_in=resid, bias=self._o_bias_full[i],
                                            eps=cfg.rms_eps)
            nxt = self.layers[i + 1].input_norm if i + 1 < len(self.layers) else self.final_norm
            if cfg.is_moe and self._moe.mode == "ep" and rows >= self.MOE_A2A_MIN_TOKENS:
                # tokens stay sharded: route this rank's rows, exchange them with the expert owners
                dn = self._moe.forward_sharded(lw, normed)
            elif cfg.is_moe:
                # few tokens: replicate them, run the local experts, sum over ranks (library collectives)
                full = tp.all_gather(normed).reshape(T, cfg.hidden_size)
                y_sorted, plan, weights = self._moe._experts(lw, full)
                y = ops.moe_combine(y_sorted, plan.pair_pos, weights, T)
                dn = tp.reduce_scatter(y)
            else:
                if cfg.swiglu_limit <= 0:
                    act = ag(normed, lw.gate_up, gated=True)           # SwiGLU in the GEMM epilogue
                else:
                    act = ops.silu_mul(ag(normed, lw.gate_up), limit=cfg.swiglu_limit, alpha=cfg.swiglu_alpha)
                dn = rs(act, lw.down)
            resid, normed = ops.add_rmsnorm(dn, nxt, residual_in=resid, eps=cfg.rms_eps)
        return tp.all_gather(normed).reshape(T, cfg.hidden_size)

    def close(self) -> None:
        """Release the symmetric (peer-mapped) buffers this model set up lazily: the sequence-parallel GEMM pair
        and the expert all-to-all.  Collective: every rank of the group calls it at the same point."""
        pair = getattr(self, "_sp_ops", None)
        if pair is not None:
            pair[0].close()
            pair[1].close()
            self._sp_ops = None
        a2a = getattr(self._moe, "_a2a", None) if self._moe is not None else None
        if a2a is not None:
            a2a.close()
            self._moe._a2a = None

    # ------------------------------------------------------------------ heads
    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """Vocab-parallel logits [rows, V / tp] (bf16)."""
        return ops.linear(hidden, self.lm_head)

    def greedy(self, hidden: torch.Tensor, out_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Greedy next token ids (int32 [rows]) from final-normed hidden states; with tp > 1
        the per-rank (max, argmax) pairs are gathered and reduced like the reference's
        vocab-parallel head."""
        logits = self.logits(hidden)
        rows = hidden.shape[0]
        if self.tp.world_size == 1:
            return ops.argmax(logits, out_ids=out_ids)
        vals = torch.empty((rows,), dtype=torch.float32, device=hidden.device)
        ids = ops.argmax(logits, out_vals=vals)
        fused = getattr(self.tp, "fused", None)
        if fused is not None and rows <= fused.max_tokens:
            # (value, id) pairs exchanged over peer memory by one kernel
            return fused.argmax_exchange(vals, ids, self.tp.rank * self.vocab_local, out_ids)
        packed = torch.stack([vals, (ids + self.tp.rank * self.vocab_local).float()], dim=-1)  # [rows, 2]
        allp = self.tp.all_gather(packed)                                                       # [tp, rows, 2]
        best = allp[..., 0].argmax(dim=0)                                                       # first max wins
        res = allp[..., 1].gather(0, best[None]).squeeze(0).to(torch.int32)
        if out_ids is not None:
            out_ids.copy_(res)
            return out_ids
        return res
