"""Text-embedding model: a prefill-only pass of the decoder, last-token pooling, L2 normalisation.

The reference pads every sequence to `max_model_len`, runs per-layer device kernels without a KV cache
and pools the last valid token on the host (examples/models/qwen3_embedding/model.py:123-262,
embedding_utils.py:6-47).  Here the sequences are packed without padding into one token batch, the
blockwise attention kernel reads K/V from a scratch paged cache that the fused RoPE kernel fills, and
pooling + normalisation stay on the device.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .config import ModelConfig
from .kv_cache import BLOCK_SIZE
from .transformer import TransformerLM


def last_token_pool(hidden: torch.Tensor, q_start: torch.Tensor, q_lens: torch.Tensor) -> torch.Tensor:
    """hidden [T, H] of packed sequences -> the row of each sequence's last token [B, H]."""
    return hidden[(q_start + q_lens - 1).long()]


def normalize_embeddings(e: torch.Tensor, eps: float = 1e-12) -> torch.Tensor:
    e = e.float()
    return e / e.norm(dim=-1, keepdim=True).clamp_min(eps)


def get_detailed_instruct(task_description: str, query: str) -> str:
    return f"Instruct: {task_description}\nQuery: {query}"


class EmbeddingModel:
    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], device, max_batch: int = 32,
                 max_model_len: int = 512):
        self.cfg = cfg
        self.device = torch.device(device)
        self.lm = TransformerLM(cfg, weights, device=device)
        self.max_batch, self.max_model_len = max_batch, max_model_len
        blocks_per_seq = (max_model_len + BLOCK_SIZE - 1) // BLOCK_SIZE
        self.cache = self.lm.new_cache(max_batch * blocks_per_seq + 1, max_batch, max_model_len,
                                       enable_prefix_sharing=False)

    @torch.no_grad()
    def encode(self, token_ids: Sequence[Sequence[int]], normalize: bool = True) -> torch.Tensor:
        """token_ids: B sequences (each truncated to max_model_len) -> embeddings fp32 [B, H]."""
        out: List[torch.Tensor] = []
        for i in range(0, len(token_ids), self.max_batch):
            out.append(self._encode_batch([list(t)[: self.max_model_len] for t in token_ids[i:i + self.max_batch]]))
        e = torch.cat(out)
        return normalize_embeddings(e) if normalize else e.float()

    def _encode_batch(self, seqs_tokens: List[List[int]]) -> torch.Tensor:
        cache, dev = self.cache, self.device
        seqs = [cache.add_sequence(t) for t in seqs_tokens]
        try:
            lens = [len(t) for t in seqs_tokens]
            ids = torch.tensor([t for s in seqs_tokens for t in s], dtype=torch.int32, device=dev)
            pos = torch.cat([torch.arange(0, n, dtype=torch.int32) for n in lens]).to(dev)
            slots = torch.cat([cache.slots_for(s, 0, n) for s, n in zip(seqs, lens)]).to(dev)
            q_start = torch.tensor([sum(lens[:i]) for i in range(len(lens))], dtype=torch.int32, device=dev)
            q_lens = torch.tensor(lens, dtype=torch.int32, device=dev)
            rows = torch.tensor([s.slot for s in seqs], dtype=torch.long, device=dev)
            hidden = self.lm.prefill(ids, pos, slots, cache, cache.block_table[rows], q_start, q_lens, q_lens,
                                     max(lens))
            return last_token_pool(hidden, q_start, q_lens).float()
        finally:
            for s in seqs:
                cache.free_sequence(s)
