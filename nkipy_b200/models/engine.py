"""Generation engine: batched prefill + CUDA-graph decode over a paged KV cache.

Plays the role of the reference's ``generate()`` loops
(examples/models/qwen3/qwen3.py:262-447: prefill, then a double-buffered decode
loop whose next-token id never leaves the device, while the previous token is
read back for the caller) and of its evaluation harness
(examples/models/qwen3/evaluate.py:107-136: TTFT, decode latency percentiles,
tokens/s).  On B200 the per-token work is one captured graph: device-side
bookkeeping (positions, cache slots, context lengths) -> embedding -> layers ->
vocab-parallel greedy head -> the new ids feed the next replay directly.
"""

from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from .kv_cache import BLOCK_SIZE, PagedKVCache, SequenceState
from .transformer import TransformerLM


def percentile(values: Sequence[float], q: float) -> float:
    """Linear-interpolation percentile (q in [0, 100])."""
    if not values:
        return float("nan")
    xs = sorted(values)
    if len(xs) == 1:
        return xs[0]
    pos = (len(xs) - 1) * q / 100.0
    lo = int(pos)
    hi = min(lo + 1, len(xs) - 1)
    return xs[lo] + (xs[hi] - xs[lo]) * (pos - lo)


@dataclass
class GenerationStats:
    ttft_s: List[float] = field(default_factory=list)
    decode_step_ms: List[float] = field(default_factory=list)
    prefill_tokens: int = 0
    cached_tokens: int = 0
    decode_tokens: int = 0
    decode_time_s: float = 0.0

    def summary(self) -> Dict[str, float]:
        return {
            "ttft_p50_s": percentile(self.ttft_s, 50),
            "ttft_p90_s": percentile(self.ttft_s, 90),
            "decode_ms_p50": percentile(self.decode_step_ms, 50),
            "decode_ms_p90": percentile(self.decode_step_ms, 90),
            "decode_ms_p99": percentile(self.decode_step_ms, 99),
            "decode_tokens_per_s": self.decode_tokens / self.decode_time_s if self.decode_time_s > 0 else 0.0,
            "prefill_tokens": self.prefill_tokens,
            "cached_tokens": self.cached_tokens,
        }


class GenerationEngine:
    """Owns the KV cache and the static decode buffers of one model replica."""

    def __init__(self, model: TransformerLM, max_batch: int, max_seq_len: int, num_blocks: Optional[int] = None,
                 prefill_chunk_tokens: int = 16384, use_cuda_graph: Optional[bool] = None,
                 enable_prefix_sharing: bool = True):
        self.model = model
        self.device = model.device
        self.max_batch = max_batch
        self.max_seq_len = max_seq_len
        blocks_per_seq = (max_seq_len + BLOCK_SIZE - 1) // BLOCK_SIZE
        if num_blocks is None:
            num_blocks = max_batch * blocks_per_seq + 8
        self.cache: PagedKVCache = model.new_cache(num_blocks, max_batch, max_seq_len, enable_prefix_sharing)
        self.prefill_chunk_tokens = prefill_chunk_tokens
        self.use_cuda_graph = (self.device.type == "cuda") if use_cuda_graph is None else use_cuda_graph
        dev = self.device
        B = max_batch
        self.ids = torch.zeros((B,), dtype=torch.int32, device=dev)
        self.positions = torch.zeros((B,), dtype=torch.int32, device=dev)
        self.slots = torch.full((B,), -1, dtype=torch.int32, device=dev)
        self.context_lens = torch.full((B,), -1, dtype=torch.int32, device=dev)   # -1 = inactive row
        pin = dev.type == "cuda"
        self.ids_host = torch.zeros((B,), dtype=torch.int32, pin_memory=pin)
        self.out_host = torch.zeros((B,), dtype=torch.int32, pin_memory=pin)
        self.active: Dict[int, SequenceState] = {}     # table row -> sequence
        self._graph = None
        tp = model.tp
        if ((tp.world_size > 1 or getattr(model, "force_fused", False)) and dev.type == "cuda"
                and getattr(tp, "fused", None) is None
                and os.environ.get("NKIPY_B200_FUSED_TP", "1") == "1"):
            from ..parallel.symm import FusedTP

            tp.fused = FusedTP(tp, max_batch, model.cfg.hidden_size)
        self.stats = GenerationStats()

    # ------------------------------------------------------------------ admission + prefill
    def add_requests(self, prompts: Sequence[Sequence[int]]) -> List[SequenceState]:
        seqs = [self.cache.add_sequence(p) for p in prompts]
        for s in seqs:
            self.active[s.slot] = s
        return seqs

    def prefill(self, seqs: Sequence[SequenceState]) -> torch.Tensor:
        """Run the uncached part of the prompts (chunked by token budget); returns the first
        generated token of every sequence (int32, device) and records per-sequence TTFT."""
        m, cache, dev = self.model, self.cache, self.device
        first = torch.zeros((len(seqs),), dtype=torch.int32, device=dev)
        t0 = time.perf_counter()
        i = 0
        while i < len(seqs):
            chunk, tok = [], 0
            while i < len(seqs) and (not chunk or tok + len(seqs[i].tokens) - seqs[i].num_cached
                                     <= self.prefill_chunk_tokens):
                chunk.append((i, seqs[i]))
                tok += len(seqs[i].tokens) - seqs[i].num_cached
                i += 1
            ids, pos, slots, q_start, q_lens, ctx, rows = [], [], [], [], [], [], []
            off = 0
            for _, s in chunk:
                n, c = len(s.tokens), s.num_cached
                ids.append(torch.tensor(s.tokens[c:], dtype=torch.int32))
                pos.append(torch.arange(c, n, dtype=torch.int32))
                slots.append(cache.slots_for(s, c, n))
                q_start.append(off)
                q_lens.append(n - c)
                ctx.append(n)
                rows.append(s.slot)
                off += n - c
            to = lambda xs, cat=True: (torch.cat(xs) if cat else torch.tensor(xs, dtype=torch.int32)).to(
                dev, non_blocking=True)
            ids_d, pos_d, slots_d = to(ids), to(pos), to(slots)
            qs_d, ql_d, ctx_d = to(q_start, False), to(q_lens, False), to(ctx, False)
            table = cache.block_table[torch.tensor(rows, dtype=torch.long, device=dev)]
            hidden = m.prefill(ids_d, pos_d, slots_d, cache, table, qs_d, ql_d, ctx_d, max(q_lens))
            last = (qs_d + ql_d - 1).long()
            tok_ids = m.greedy(hidden[last].contiguous())
            for j, (gi, s) in enumerate(chunk):
                first[gi:gi + 1].copy_(tok_ids[j:j + 1])
            if dev.type == "cuda":
                torch.cuda.synchronize()
            done = time.perf_counter() - t0
            for _, s in chunk:
                self.stats.ttft_s.append(done)
                self.stats.prefill_tokens += len(s.tokens) - s.num_cached
                self.stats.cached_tokens += s.num_cached
                cache.mark_computed(s, len(s.tokens))
        # seed the decode buffers
        host_first = first.cpu()
        for j, s in enumerate(seqs):
            self.ids_host[s.slot] = host_first[j]
            s.tokens.append(int(host_first[j]))
        self._sync_rows(seqs)
        return first

    def _sync_rows(self, seqs: Sequence[SequenceState]) -> None:
        """Push ids / context lengths of the given rows to the device buffers."""
        ctx_host = self.context_lens.cpu()
        for s in seqs:
            ctx_host[s.slot] = s.num_computed
        self.context_lens.copy_(ctx_host)
        self.ids.copy_(self.ids_host, non_blocking=True)

    # ------------------------------------------------------------------ decode
    def _reserve(self, steps: int) -> None:
        """Blocks for the next `steps` tokens of every active sequence (host-side)."""
        for s in self.active.values():
            need = s.num_computed + steps + 1
            if need > self.max_seq_len:
                raise RuntimeError(f"sequence would exceed max_seq_len={self.max_seq_len}")
            self.cache.ensure_capacity(s, need)

    def _decode_body(self) -> None:
        m = self.model
        fused = getattr(m.tp, "fused", None)
        if fused is not None:
            fused.begin_step()
        ops.decode_advance(self.context_lens, self.cache.block_table, self.positions, self.slots, 1, BLOCK_SIZE)
        hidden = m.decode_step(self.ids, self.positions, self.slots, self.cache, self.cache.block_table,
                               self.context_lens)
        m.greedy(hidden, out_ids=self.ids)

    def _ensure_graph(self) -> None:
        if not self.use_cuda_graph or self._graph is not None:
            return
        # warm up on a side stream (allocations, attribute setup, NCCL channels), restoring the
        # state the warm-up step mutates, then capture
        saved = (self.ids.clone(), self.context_lens.clone())
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                self._decode_body()
                self.ids.copy_(saved[0])
                self.context_lens.copy_(saved[1])
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        before = ops.launch_count()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._decode_body()
        self.launches_per_step = ops.launch_count() - before
        self.ids.copy_(saved[0])
        self.context_lens.copy_(saved[1])
        torch.cuda.synchronize()
        self._graph = g

    def decode_step_device(self) -> None:
        """One decode step whose input ids are already on the device (the previous step's
        output); nothing crosses PCIe."""
        if self.use_cuda_graph:
            self._graph.replay()
        else:
            self._decode_body()

    def step(self, ids_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Public per-step API: token ids in pinned host memory -> device, one decode step,
        new ids back to pinned host memory (synchronises).  Without ids_host the ids already on
        the device are used."""
        if ids_host is not None:
            self.ids.copy_(ids_host, non_blocking=True)
        self.decode_step_device()
        self.out_host.copy_(self.ids, non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        return self.out_host

    def prepare_decode(self, steps: int) -> None:
        self._reserve(steps)
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        self._ensure_graph()

    def advance_host_state(self, steps: int, new_tokens: Optional[torch.Tensor] = None) -> None:
        for s in self.active.values():
            s.num_computed += steps

    # ------------------------------------------------------------------ top-level API
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, eos_token_id: Optional[int] = None
                 ) -> List[List[int]]:
        """Greedy generation for a batch of prompts; returns the new token ids per prompt."""
        seqs = self.add_requests(prompts)
        self.prefill(seqs)
        outs: List[List[int]] = [[s.tokens[-1]] for s in seqs]
        finished = [eos_token_id is not None and o[0] == eos_token_id for o in outs]
        if max_new_tokens > 1:
            self.prepare_decode(max_new_tokens)
        t0 = time.perf_counter()
        steps = 0
        for _ in range(max_new_tokens - 1):
            if all(finished):
                break
            ts = time.perf_counter()
            host = self.step().clone()
            self.stats.decode_step_ms.append((time.perf_counter() - ts) * 1e3)
            self.advance_host_state(1)
            steps += 1
            for j, s in enumerate(seqs):
                if finished[j]:
                    continue
                tok = int(host[s.slot])
                outs[j].append(tok)
                s.tokens.append(tok)
                if eos_token_id is not None and tok == eos_token_id:
                    finished[j] = True
        self.stats.decode_time_s += time.perf_counter() - t0
        self.stats.decode_tokens += steps * len(seqs)
        self.release(seqs)
        return outs

    def release(self, seqs: Sequence[SequenceState]) -> None:
        ctx_host = self.context_lens.cpu()
        for s in seqs:
            ctx_host[s.slot] = -1
            self.active.pop(s.slot, None)
            self.cache.free_sequence(s)
        self.context_lens.copy_(ctx_host)
