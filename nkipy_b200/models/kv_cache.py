"""Paged KV cache: block allocator with reference counts and prefix sharing.

The reference keeps one dense ``[B, max_seq_len, kv_heads, head_dim]`` cache per
layer that kernels alias in place (examples/models/qwen3/qwen3.py:52-71).  Here
the cache is a pool of 32-token blocks per layer, laid out
``[num_blocks, kv_heads, 32, head_dim]`` so that one (block, head) page is a
contiguous slab for TMA; sequences own lists of block ids (the block table).
Full blocks are content-addressed by the hash of their token ids chained with
the hash of the preceding block, so sequences with a common prompt prefix share
the blocks (reference-counted; a freed block stays findable until it is
recycled, least recently freed first).
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

BLOCK_SIZE = 32


class OutOfBlocks(RuntimeError):
    pass


@dataclass
class SequenceState:
    seq_id: int
    tokens: List[int]
    blocks: List[int] = field(default_factory=list)
    num_cached: int = 0      # tokens whose K/V were found in shared blocks at admission
    num_computed: int = 0    # tokens whose K/V are in the cache
    slot: int = -1           # row of the batch tables this sequence occupies


class BlockAllocator:
    """Host-side block bookkeeping (no device work)."""

    def __init__(self, num_blocks: int, block_size: int = BLOCK_SIZE, enable_prefix_sharing: bool = True):
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.enable_prefix_sharing = enable_prefix_sharing
        self.ref = [0] * num_blocks
        self.free: List[int] = list(range(num_blocks - 1, -1, -1))
        self.hash_of: List[Optional[int]] = [None] * num_blocks
        self.by_hash: Dict[int, int] = {}
        self.evictable: "OrderedDict[int, None]" = OrderedDict()  # ref == 0 but content still valid

    # -- capacity
    def num_free(self) -> int:
        return len(self.free) + len(self.evictable)

    def _take(self) -> int:
        if self.free:
            b = self.free.pop()
        elif self.evictable:
            b, _ = self.evictable.popitem(last=False)
            h = self.hash_of[b]
            if h is not None and self.by_hash.get(h) == b:
                del self.by_hash[h]
            self.hash_of[b] = None
        else:
            raise OutOfBlocks("KV cache exhausted")
        self.ref[b] = 1
        return b

    def _share(self, b: int) -> None:
        if self.ref[b] == 0:
            self.evictable.pop(b, None)
        self.ref[b] += 1

    @staticmethod
    def chain_hash(parent: Optional[int], tokens: Sequence[int]) -> int:
        return hash((parent, tuple(tokens)))

    # -- sequence lifecycle
    def admit(self, tokens: Sequence[int]) -> Tuple[List[int], int]:
        """Blocks for a new sequence holding `tokens`.  Returns (block ids, number of
        leading tokens whose K/V are already cached in shared blocks).  At least one
        token is always left to compute so the sequence produces logits."""
        bs = self.block_size
        n = len(tokens)
        blocks: List[int] = []
        cached = 0
        parent: Optional[int] = None
        nfull = n // bs
        if self.enable_prefix_sharing:
            for i in range(nfull):
                if (i + 1) * bs >= n:  # keep the last token uncached
                    break
                h = self.chain_hash(parent, tokens[i * bs:(i + 1) * bs])
                b = self.by_hash.get(h)
                if b is None:
                    break
                self._share(b)
                blocks.append(b)
                cached += bs
                parent = h
        need = (n + bs - 1) // bs - len(blocks)
        if need > self.num_free():
            for b in blocks:
                self.release_block(b)
            raise OutOfBlocks(f"need {need} blocks, {self.num_free()} free")
        for _ in range(need):
            blocks.append(self._take())
        return blocks, cached

    def publish(self, tokens: Sequence[int], blocks: Sequence[int], upto: int) -> None:
        """Make the full blocks covering tokens[:upto] findable for prefix sharing
        (called once their K/V have been written)."""
        if not self.enable_prefix_sharing:
            return
        bs = self.block_size
        parent: Optional[int] = None
        for i in range(upto // bs):
            h = self.chain_hash(parent, tokens[i * bs:(i + 1) * bs])
            b = blocks[i]
            if self.hash_of[b] is None and h not in self.by_hash:
                self.hash_of[b] = h
                self.by_hash[h] = b
            parent = h

    def extend(self, blocks: List[int], new_len: int) -> int:
        """Grow a block list to cover new_len tokens; returns the number of blocks added."""
        need = (new_len + self.block_size - 1) // self.block_size - len(blocks)
        for _ in range(max(need, 0)):
            blocks.append(self._take())
        return max(need, 0)

    def release_block(self, b: int) -> None:
        self.ref[b] -= 1
        if self.ref[b] < 0:
            raise RuntimeError(f"block {b} released twice")
        if self.ref[b] == 0:
            if self.hash_of[b] is not None:
                self.evictable[b] = None
            else:
                self.free.append(b)

    def release(self, blocks: Sequence[int]) -> None:
        for b in blocks:
            self.release_block(b)


class PagedKVCache:
    """Per-layer K/V block pools plus the batch-level device tables the kernels read."""

    def __init__(self, num_layers: int, num_kv_heads: int, head_dim: int, num_blocks: int, max_batch: int,
                 max_blocks_per_seq: int, device, dtype=torch.bfloat16, enable_prefix_sharing: bool = True):
        self.num_layers = num_layers
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.block_size = BLOCK_SIZE
        self.num_blocks = num_blocks
        self.max_batch = max_batch
        self.max_blocks_per_seq = max_blocks_per_seq
        self.device = torch.device(device)
        shape = (num_blocks, num_kv_heads, BLOCK_SIZE, head_dim)
        # zero-filled: masked positions are multiplied by probability 0 and must be finite
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.allocator = BlockAllocator(num_blocks, BLOCK_SIZE, enable_prefix_sharing)
        self.block_table = torch.zeros((max_batch, max_blocks_per_seq), dtype=torch.int32, device=device)
        pin = self.device.type == "cuda"
        self._table_host = torch.zeros((max_batch, max_blocks_per_seq), dtype=torch.int32, pin_memory=pin)
        self.sequences: Dict[int, SequenceState] = {}
        self._free_slots = list(range(max_batch - 1, -1, -1))
        self._next_id = 0

    def bytes(self) -> int:
        per = self.k[0].numel() * self.k[0].element_size()
        return 2 * per * self.num_layers

    # -- admission / growth / release
    def add_sequence(self, tokens: Sequence[int]) -> SequenceState:
        if not self._free_slots:
            raise OutOfBlocks("batch table full")
        blocks, cached = self.allocator.admit(tokens)
        if len(blocks) > self.max_blocks_per_seq:
            self.allocator.release(blocks)
            raise OutOfBlocks("sequence longer than max_blocks_per_seq")
        seq = SequenceState(self._next_id, list(tokens), blocks, cached, cached, self._free_slots.pop())
        self._next_id += 1
        self.sequences[seq.seq_id] = seq
        self._write_row(seq)
        return seq

    def ensure_capacity(self, seq: SequenceState, new_len: int) -> bool:
        """Make sure the sequence has blocks for new_len tokens; True when the table changed."""
        if (new_len + BLOCK_SIZE - 1) // BLOCK_SIZE > self.max_blocks_per_seq:
            raise OutOfBlocks("sequence longer than max_blocks_per_seq")
        added = self.allocator.extend(seq.blocks, new_len)
        if added:
            self._write_row(seq)
        return added > 0

    def mark_computed(self, seq: SequenceState, upto: int) -> None:
        seq.num_computed = upto
        self.allocator.publish(seq.tokens, seq.blocks, min(upto, len(seq.tokens)))

    def free_sequence(self, seq: SequenceState) -> None:
        self.allocator.release(seq.blocks)
        seq.blocks = []
        self._free_slots.append(seq.slot)
        self.sequences.pop(seq.seq_id, None)

    def _write_row(self, seq: SequenceState) -> None:
        row = self._table_host[seq.slot]
        n = len(seq.blocks)
        row[:n] = torch.tensor(seq.blocks, dtype=torch.int32)
        self.block_table[seq.slot, :n].copy_(row[:n], non_blocking=True)

    def slots_for(self, seq: SequenceState, start: int, end: int) -> torch.Tensor:
        """Flat cache slots (block * block_size + offset) of token positions [start, end)."""
        pos = torch.arange(start, end, dtype=torch.int64)
        blocks = torch.tensor(seq.blocks, dtype=torch.int64)
        return (blocks[pos // BLOCK_SIZE] * BLOCK_SIZE + pos % BLOCK_SIZE).to(torch.int32)
