"""Parallel-drafting speculative decoding (P-EAGLE style) on the paged engine.

A small replicated *drafter* proposes K tokens per step in ONE forward pass and the target verifies
them in one (K + 1)-token decode step; the longest matching prefix plus the target's own next token
is emitted, so greedy output is identical to plain decoding whatever the drafter proposes.

Drafter (examples/models/gpt_oss/peagle/drafter_model.py:175-345, kernels/drafter.py:23-174 in the
reference): 4 Llama layers over its own KV cache.  Row p of the drafter holds the pair
(embedding of token p + 1, fc(target hidden states at position p, tapped after three layers)); the
first ("fusion") layer normalises both halves separately and feeds their concatenation (2H wide) to
its attention, using the hidden half as the residual.  A step processes
``[commit_0 .. commit_{C-1} | ptd_0 .. ]`` rows per sequence: the C tokens the target accepted last
step (with their real target hidden states) followed by placeholder rows (a fixed "ptd" token
embedding and the learned ``mask_hidden``); the drafts are the arg-max of rows C - 1 .. C + K - 2,
mapped from the drafter's reduced vocabulary with the ``d2t`` offsets.  Every sequence is padded to
the fixed window W = 2K, as the reference pads to its single compiled kernel.

Rollback is implicit in both caches: rejected rows are overwritten at their absolute positions by
the next step and the causal mask hides rows past a query's position
(examples/models/gpt_oss/peagle/speculate.py:16-18).

Differences from the reference: batched (B sequences per step, each with its own acceptance count),
paged KV caches sharing one block table, the embedding gather, arg-max and d2t remap stay on the
device, and the target's tap hidden states never leave the GPU.
"""

from __future__ import annotations

import dataclasses
import time
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from .config import ModelConfig
from .kv_cache import BLOCK_SIZE, PagedKVCache
from .transformer import TransformerLM
from .weights import random_weights, to_device_layout


@dataclasses.dataclass
class EagleConfig:
    """Shape of the drafter (examples/models/gpt_oss/peagle/config.py:12-83 in the reference)."""
    hidden_size: int
    target_hidden_size: int
    num_layers: int = 4
    num_heads: int = 8
    num_kv_heads: int = 8
    head_dim: int = 64
    intermediate_size: int = 1024
    draft_vocab_size: int = 512
    vocab_size: int = 512
    ptd_token_id: int = 0
    num_draft_tokens: int = 3
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_position: int = 4096

    def model_config(self) -> ModelConfig:
        return ModelConfig(name="eagle-drafter", vocab_size=self.draft_vocab_size, hidden_size=self.hidden_size,
                           num_layers=self.num_layers, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                           head_dim=self.head_dim, intermediate_size=self.intermediate_size,
                           max_position=self.max_position, rms_eps=self.rms_eps, rope_theta=self.rope_theta)


def tap_layers(num_layers: int):
    """Target layers whose output feeds the drafter: early, middle, late
    (examples/models/gpt_oss/peagle/config.py:47-58)."""
    return (min(1, num_layers - 1), max(0, num_layers // 2 - 1), max(0, num_layers - 4))


def random_drafter_weights(ecfg: EagleConfig, device="cpu", seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Random drafter in the same schema as the target's weights plus the drafter-only tensors."""
    cfg = ecfg.model_config()
    w = random_weights(cfg, 0, 1, device=device, seed=seed, std=std)
    H, tH = ecfg.hidden_size, ecfg.target_hidden_size
    g = torch.Generator().manual_seed(seed * 7919 + 5)
    rnd = lambda *shape: (torch.randn(*shape, generator=g) * std).to(torch.bfloat16).to(device)
    # fusion layer: attention reads cat(norm(embed), norm(hidden)) of width 2H
    w["layers.0.qkv_weight"] = rnd(2 * H, cfg.q_size + 2 * cfg.kv_size)
    w["layers.0.hidden_norm_weight"] = torch.ones(H, dtype=torch.bfloat16, device=device)
    w["fc_weight"] = rnd(3 * tH, H)
    w["mask_hidden"] = rnd(3 * tH)
    w["embed_tokens"] = rnd(ecfg.vocab_size, H)
    w["d2t"] = torch.zeros(ecfg.draft_vocab_size, dtype=torch.int64, device=device)
    return w


class DrafterLM:
    """The drafter on the kernel library: a 4-layer `TransformerLM` whose first layer is fed by hand."""

    def __init__(self, ecfg: EagleConfig, weights: Dict[str, torch.Tensor], device):
        self.ecfg = ecfg
        self.device = torch.device(device)
        self.lm = TransformerLM(ecfg.model_config(), weights, device=device)
        dev = self.device
        self.fc = to_device_layout(weights["fc_weight"].to(dev))                  # [H, 3 tH]
        self.mask_hidden = weights["mask_hidden"].to(dev).reshape(1, -1).contiguous()
        self.hidden_norm = weights["layers.0.hidden_norm_weight"].to(dev)
        self.embed_tokens = weights["embed_tokens"].to(dev).contiguous()
        self.d2t = weights["d2t"].to(dev).to(torch.int64)
        self._mask_fused = None

    def new_cache(self, like: PagedKVCache) -> PagedKVCache:
        """A cache with the target's geometry, so both models share one block table."""
        cfg = self.lm.cfg
        return PagedKVCache(cfg.num_layers, self.lm.nkv, self.lm.d, like.num_blocks, like.max_batch,
                            like.max_blocks_per_seq, self.device, enable_prefix_sharing=False)

    def _inputs(self, token_ids: torch.Tensor, hidden3: torch.Tensor, is_mask: Optional[torch.Tensor]):
        """(residual, first-layer input) for rows with token ids [T] and tap hiddens [T, 3 tH]; rows
        flagged in is_mask use the shared fc(mask_hidden) instead."""
        eps = self.ecfg.rms_eps
        emb = ops.embedding(token_ids, self.embed_tokens)
        hid = ops.linear(hidden3, self.fc)
        if is_mask is not None:
            if self._mask_fused is None:
                self._mask_fused = ops.linear(self.mask_hidden, self.fc)
            hid = torch.where(is_mask[:, None], self._mask_fused.expand_as(hid), hid)
        e_n = ops.rmsnorm(emb, self.lm.layers[0].input_norm, eps)
        h_n = ops.rmsnorm(hid, self.hidden_norm, eps)
        return hid, torch.cat([e_n, h_n], dim=-1).contiguous()

    def prefill(self, token_ids, hidden3, positions, slots, cache, block_table, q_start, q_lens, context_lens,
                max_q_len):
        inputs = self._inputs(token_ids, hidden3, None)
        return self.lm.prefill(token_ids, positions, slots, cache, block_table, q_start, q_lens, context_lens,
                               max_q_len, inputs=inputs)

    def step(self, token_ids, hidden3, is_mask, positions, slots, cache, block_table, context_lens, q_len):
        """One drafting pass over q_len rows per sequence; returns draft-vocabulary logits [B * q_len, Vd]."""
        inputs = self._inputs(token_ids, hidden3, is_mask)
        h = self.lm.decode_step(token_ids, positions, slots, cache, block_table, context_lens, q_len=q_len,
                                inputs=inputs)
        return self.lm.logits(h)


@dataclasses.dataclass
class SpecStats:
    steps: int = 0
    emitted: int = 0
    draft_s: float = 0.0
    verify_s: float = 0.0
    ttft_s: float = 0.0
    decode_s: float = 0.0

    @property
    def mean_acceptance(self) -> float:
        return self.emitted / max(1, self.steps)


class SpeculativeEngine:
    """Target engine state + drafter + the accept loop (examples/models/gpt_oss/peagle/speculate.py:236-459)."""

    def __init__(self, target: TransformerLM, drafter: DrafterLM, max_batch: int, max_seq_len: int,
                 num_draft_tokens: Optional[int] = None, num_blocks: Optional[int] = None):
        if target.tp.world_size != 1:
            raise NotImplementedError("speculative decoding runs the target on one rank here")
        self.target, self.drafter = target, drafter
        self.K = num_draft_tokens or drafter.ecfg.num_draft_tokens
        self.W = 2 * self.K                                 # fixed drafter window, as in the reference
        self.dev = target.device
        self.max_batch, self.max_seq_len = max_batch, max_seq_len
        slack = self.W + self.K + 2                          # speculative rows past the committed length
        blocks_per_seq = (max_seq_len + slack + BLOCK_SIZE - 1) // BLOCK_SIZE
        if num_blocks is None:
            num_blocks = max_batch * blocks_per_seq + 1
        self.cache = target.new_cache(num_blocks, max_batch, max_seq_len + slack, enable_prefix_sharing=False)
        self.dcache = drafter.new_cache(self.cache)
        self.taps = tap_layers(target.cfg.num_layers)
        self.stats = SpecStats()

    # ------------------------------------------------------------------ helpers
    def _slots(self, seqs, starts: Sequence[int], n: int) -> torch.Tensor:
        return torch.cat([self.cache.slots_for(s, st, st + n) for s, st in zip(seqs, starts)]).to(self.dev)

    def _aux3(self, taps: List[torch.Tensor]) -> torch.Tensor:
        return torch.cat([taps[i] for i in self.taps], dim=-1).contiguous()

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int) -> List[List[int]]:
        K, W, dev = self.K, self.W, self.dev
        tgt, dr, cache = self.target, self.drafter, self.cache
        B = len(prompts)
        if B > self.max_batch:
            raise ValueError("more prompts than max_batch")
        seqs = [cache.add_sequence(p) for p in prompts]
        for s in seqs:
            cache.ensure_capacity(s, min(len(s.tokens) + max_new_tokens + W + K + 2,
                                         cache.max_blocks_per_seq * BLOCK_SIZE))
        rows = torch.tensor([s.slot for s in seqs], dtype=torch.long, device=dev)
        table = cache.block_table[rows]
        t0 = time.perf_counter()

        # ---- target prefill with taps, first token
        lens = [len(p) for p in prompts]
        ids = torch.tensor([t for p in prompts for t in p], dtype=torch.int32, device=dev)
        pos = torch.cat([torch.arange(0, n, dtype=torch.int32) for n in lens]).to(dev)
        slots = torch.cat([cache.slots_for(s, 0, n) for s, n in zip(seqs, lens)]).to(dev)
        q_start = torch.tensor([sum(lens[:i]) for i in range(B)], dtype=torch.int32, device=dev)
        q_lens = torch.tensor(lens, dtype=torch.int32, device=dev)
        hidden, taps = tgt.prefill(ids, pos, slots, cache, table, q_start, q_lens, q_lens, max(lens),
                                   return_hidden=True)
        last = (q_start + q_lens - 1).long()
        first = tgt.greedy(hidden[last].contiguous())
        # ---- drafter prefill: row p = (token p + 1, target hidden p)
        shifted = ids.clone()
        shifted[:-1] = ids[1:]
        shifted[last] = first
        dr.prefill(shifted, self._aux3(taps), pos, slots, self.dcache, table, q_start, q_lens, q_lens, max(lens))
        first_h = first.cpu().tolist()
        if dev.type == "cuda":
            torch.cuda.synchronize()
        self.stats.ttft_s = time.perf_counter() - t0

        out: List[List[int]] = [[t] for t in first_h]
        L = list(lens)                         # tokens whose KV is in the target cache, per sequence
        # pending commit for the drafter: the last C emitted tokens and the target hiddens that produced them
        commit_tok = [[t] for t in first_h]
        commit_aux = [self._aux3(taps)[last[b]:last[b] + 1] for b in range(B)]
        t_dec = time.perf_counter()
        ptd = dr.ecfg.ptd_token_id
        tH3 = commit_aux[0].shape[-1]

        # A sequence that has its max_new_tokens is frozen: it stays in the batch (static shapes), but its
        # committed length, pending commit and output no longer advance, so its speculative rows keep
        # landing on the same reserved cache slots however long the slowest sequence still needs.
        done = [len(o) >= max_new_tokens for o in out]
        while not all(done):
            # ---- draft: window of W rows per sequence starting at base = L - C + ... (position of commit_0)
            t1 = time.perf_counter()
            tok_rows = torch.full((B, W), ptd, dtype=torch.int32)
            is_mask = torch.ones((B, W), dtype=torch.bool)
            aux = torch.zeros((B, W, tH3), dtype=torch.bfloat16, device=dev)
            base, Cs = [], []
            for b in range(B):
                C = len(commit_tok[b])
                Cs.append(C)
                base.append(L[b] - C + 0)        # row 0 sits at the position of the hidden that produced commit_0
                tok_rows[b, :C] = torch.tensor(commit_tok[b], dtype=torch.int32)
                is_mask[b, :C] = False
                aux[b, :C] = commit_aux[b]
            base_pos = [L[b] - Cs[b] for b in range(B)]
            d_pos = torch.cat([torch.arange(bp, bp + W, dtype=torch.int32) for bp in base_pos]).to(dev)
            d_slots = self._slots(seqs, base_pos, W)
            d_ctx = torch.tensor([bp + W for bp in base_pos], dtype=torch.int32, device=dev)
            logits = dr.step(tok_rows.reshape(-1).to(dev), aux.reshape(B * W, tH3), is_mask.reshape(-1).to(dev),
                             d_pos, d_slots, self.dcache, table, d_ctx, W)
            local = ops.argmax(logits).long()
            draft_all = (local + dr.d2t[local]).reshape(B, W)
            sel = torch.tensor([[Cs[b] - 1 + i for i in range(K)] for b in range(B)], dtype=torch.long, device=dev)
            drafts = draft_all.gather(1, sel).to(torch.int32)                      # [B, K]
            if dev.type == "cuda":
                torch.cuda.synchronize()
            self.stats.draft_s += time.perf_counter() - t1

            # ---- verify: [last emitted, d_1 .. d_K] at positions L .. L + K
            t2 = time.perf_counter()
            last_tok = torch.tensor([o[-1] for o in out], dtype=torch.int32, device=dev)
            v_ids = torch.cat([last_tok[:, None], drafts], dim=1).reshape(-1).contiguous()
            v_pos = torch.cat([torch.arange(l, l + K + 1, dtype=torch.int32) for l in L]).to(dev)
            v_slots = self._slots(seqs, L, K + 1)
            v_ctx = torch.tensor([l + K + 1 for l in L], dtype=torch.int32, device=dev)
            h, vtaps = tgt.decode_step(v_ids, v_pos, v_slots, cache, table, v_ctx, q_len=K + 1, return_hidden=True)
            pred = tgt.greedy(h).reshape(B, K + 1)                                 # pred[:, i] follows row i
            match = (pred[:, :K] == drafts).to(torch.int32)
            n_acc = match.cumprod(dim=1).sum(dim=1)                                # accepted drafts per sequence
            pred_h, n_acc_h = pred.cpu().tolist(), n_acc.cpu().tolist()
            aux_all = self._aux3(vtaps).reshape(B, K + 1, tH3)
            self.stats.verify_s += time.perf_counter() - t2

            for b in range(B):
                if done[b]:
                    continue
                j = n_acc_h[b]
                emitted = pred_h[b][:j + 1]                # j matched drafts (== pred) + the target's next token
                out[b].extend(emitted)
                commit_tok[b] = emitted
                commit_aux[b] = aux_all[b, :j + 1]
                L[b] += j + 1
                self.stats.emitted += j + 1
                self.stats.steps += 1
                done[b] = len(out[b]) >= max_new_tokens
        self.stats.decode_s = time.perf_counter() - t_dec
        for s in seqs:
            cache.free_sequence(s)
        return [o[:max_new_tokens] for o in out]
