"""Expert-parallel MoE block over a token all-to-all in peer memory.

Tokens are sharded over the ranks of the group (the sequence-parallel prefill keeps one row slab per
rank; a data-parallel decode keeps its own sequences), experts are sharded too.  `MoEAllToAll.forward`
runs one MoE block for this rank's tokens:

    count + plan      this rank's per-expert pair counts go to every rank, every rank derives the same
                      placement of all (source, expert) row segments and the schedule of its own grouped GEMMs
    dispatch          each routed activation row is stored into its expert owner's receive buffer over NVLink
    grouped GEMMs     gate / up with SwiGLU, then down, on the rows received; each expert's tiles start as
                      soon as all sources have delivered that expert's rows (arrival counters in the kernel)
    combine           each token's k expert outputs are fetched back from the owners, weighted and summed

(csrc/kernels/moe_a2a.cu, csrc/kernels/gemm_tcgen05.cuh).  No library collective is involved and every
wait inside the kernels is bounded.

The reference keeps all experts on every rank, shards their width and all-reduces the block output
(examples/models/qwen3/kernels/transformer_layer.py:70-115); this is the expert-parallel form of that block.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import ops
from ..ops import _lib
from .comm import TPGroup
from .symm import SymmetricMemory

_FLAG_BYTES = 8192          # cnt_flag @ 0, ready @ 64, arrive @ 1024 (up to 1024 local experts)
_CNT_BYTES = 32768          # count matrix [ranks <= 8][experts <= 1024] int32


class MoEAllToAll:
    """Buffers and call counter of the expert-parallel all-to-all; one instance serves all layers."""

    def __init__(self, tp: TPGroup, max_local_tokens: int, top_k: int, hidden: int, num_experts: int,
                 capacity_factor: float = 2.0):
        n = tp.world_size
        if n > 8:
            raise ValueError("the expert all-to-all supports up to 8 ranks (one NVSwitch domain)")
        if num_experts % n or num_experts > 1024:
            raise ValueError("num_experts must be a multiple of the number of ranks and at most 1024")
        self.tp, self.top_k, self.hidden, self.num_experts = tp, top_k, hidden, num_experts
        self.max_local_tokens = max_local_tokens
        self.experts_local = num_experts // n
        pairs = max_local_tokens * top_k
        # rows this rank may receive: its fair share times the capacity factor (everything, with one rank)
        cap = pairs if n == 1 else int(capacity_factor * pairs)
        self.capacity_rows = max(128, (cap + 127) // 128 * 128)
        row_bytes = hidden * 2
        self._x_off = _FLAG_BYTES + _CNT_BYTES
        self._y_off = self._x_off + self.capacity_rows * row_bytes
        total = self._y_off + self.capacity_rows * row_bytes
        self.mem = SymmetricMemory(tp, total)
        P = ctypes.c_void_p
        ptrs = self.mem.ptrs
        self._cnt = (P * n)(*[p + _FLAG_BYTES for p in ptrs])
        self._cnt_flag = (P * n)(*ptrs)
        self._ready = (P * n)(*[p + 64 for p in ptrs])
        self._arrive = (P * n)(*[p + 1024 for p in ptrs])
        self._x_recv = (P * n)(*[p + self._x_off for p in ptrs])
        self._y = (P * n)(*[p + self._y_off for p in ptrs])
        self.x_recv = self.mem.view(self._x_off, self.capacity_rows * row_bytes, torch.bfloat16,
                                    (self.capacity_rows, hidden))
        self.y = self.mem.view(self._y_off, self.capacity_rows * row_bytes, torch.bfloat16,
                               (self.capacity_rows, hidden))
        self.arrive_ptr = self.mem.local_ptr + 1024
        dev = tp.device
        self.bn_a, self.bn_b = ops.moe_tile_widths(self.capacity_rows)
        el = self.experts_local
        self.cap_a = el + self.capacity_rows // self.bn_a + 1
        self.cap_b = el + self.capacity_rows // self.bn_b + 1
        work = torch.zeros((2 * num_experts + el + 1 + pairs + 2 * self.cap_a + 2 * self.cap_b + 3,),
                           dtype=torch.int32, device=dev)
        o = 0
        self.cursors = work[o:o + num_experts]; o += num_experts
        self.sent = work[o:o + num_experts]; o += num_experts
        self.offsets = work[o:o + el + 1]; o += el + 1
        self.pair_dest = work[o:o + pairs]; o += pairs
        self.tiles_a = work[o:o + 2 * self.cap_a]; o += 2 * self.cap_a
        self.tiles_b = work[o:o + 2 * self.cap_b]; o += 2 * self.cap_b
        self.ntiles = work[o:o + 2]; o += 2
        self.total_rows = work[o:o + 1]
        self._work = work
        self.epoch = 0           # dispatches so far (count flags, per-expert arrival counters)
        self.ready_epoch = 0     # combines so far ("expert outputs complete" counters)
        self._lib = _lib.lib()

    def dispatch(self, x: torch.Tensor, experts: torch.Tensor) -> None:
        """Count exchange, plan and the row all-to-all for this rank's tokens (two launches)."""
        T, H = x.shape
        k = experts.shape[1]
        if T > self.max_local_tokens or k != self.top_k or H != self.hidden:
            raise ValueError(f"MoEAllToAll sized for [{self.max_local_tokens}, {self.hidden}] x top-{self.top_k}")
        if experts.dtype != torch.int32 or not experts.is_contiguous():
            experts = experts.to(torch.int32).contiguous()
        tp, n = self.tp, self.tp.world_size
        self.epoch += 1
        rc = self._lib.nkb_moe_a2a_dispatch(
            x.data_ptr(), experts.data_ptr(), T, k, H, self.num_experts, n, tp.rank, self.epoch, self._cnt,
            self._cnt_flag, self._arrive, self._ready, self._x_recv, self._y, self.cursors.data_ptr(),
            self.sent.data_ptr(), self.offsets.data_ptr(), self.pair_dest.data_ptr(), self.capacity_rows, self.bn_a,
            self.tiles_a.data_ptr(), self.ntiles.data_ptr(), self.bn_b, self.tiles_b.data_ptr(),
            self.ntiles.data_ptr() + 4, self.total_rows.data_ptr(), torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "nkb_moe_a2a_dispatch")
        ops._launches += 2

    def run_experts(self, gate_up: torch.Tensor, down: torch.Tensor, *, gate_up_bias=None, down_bias=None,
                    act_limit: float = 0.0, act_alpha: float = 1.702) -> None:
        """The two grouped GEMMs on the received rows; the first waits per expert for the rows of the
        latest `dispatch`; the result stays in the peer-readable output buffer."""
        n = self.tp.world_size
        tiles = {self.bn_a: (self.tiles_a, self.ntiles[0:1], self.cap_a)}
        tiles.setdefault(self.bn_b, (self.tiles_b, self.ntiles[1:2], self.cap_b))
        target = (self.epoch * n) & 0xFFFFFFFF
        h = ops.grouped_linear(self.x_recv, gate_up, self.offsets, max_rows_per_group=self.capacity_rows, gated=True,
                               bias=gate_up_bias, act_limit=act_limit, act_alpha=act_alpha, tiles=tiles,
                               arrive=self.arrive_ptr, arrive_target=target)
        ops.grouped_linear(h, down, self.offsets, max_rows_per_group=self.capacity_rows, bias=down_bias, tiles=tiles,
                           out=self.y)

    def combine(self, weights: torch.Tensor, tokens: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Announce this rank's expert outputs, wait for the others', and fetch + weight + sum the k output rows
        of each of this rank's tokens (placement from the latest `dispatch`)."""
        tp, n = self.tp, self.tp.world_size
        weights = weights.contiguous()
        if out is None:
            out = torch.empty((tokens, self.hidden), dtype=torch.bfloat16, device=weights.device)
        self.ready_epoch += 1
        rc = self._lib.nkb_moe_a2a_combine(self.pair_dest.data_ptr(), weights.data_ptr(), tokens, self.top_k,
                                           self.hidden, n, tp.rank, self.ready_epoch, self._cnt, self._cnt_flag,
                                           self._arrive, self._ready, self._x_recv, self._y, out.data_ptr(),
                                           torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "nkb_moe_a2a_combine")
        ops._launches += 1
        return out

    def forward(self, x: torch.Tensor, experts: torch.Tensor, weights: torch.Tensor, gate_up: torch.Tensor,
                down: torch.Tensor, *, gate_up_bias: Optional[torch.Tensor] = None,
                down_bias: Optional[torch.Tensor] = None, act_limit: float = 0.0, act_alpha: float = 1.702,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [T_l, H] bf16: this rank's tokens; experts [T_l, k] int32 global expert ids; weights [T_l, k] fp32;
        gate_up [E_l, 2 I, H], down [E_l, H, I]: this rank's experts.  Returns sum_j w[t, j] * expert_j(x[t])
        for this rank's tokens, [T_l, H] bf16.  Every rank of the group must call it (collective)."""
        self.dispatch(x, experts)
        self.run_experts(gate_up, down, gate_up_bias=gate_up_bias, down_bias=down_bias, act_limit=act_limit,
                         act_alpha=act_alpha)
        return self.combine(weights, x.shape[0], out)

    def bytes_sent_per_rank(self, tokens: int) -> int:
        """Activation bytes that leave one rank in dispatch (the same amount comes back in combine) under
        uniform routing: every pair's row crosses NVLink unless its expert is local."""
        n = self.tp.world_size
        return int(tokens * self.top_k * self.hidden * 2 * (n - 1) / n)

    def close(self) -> None:
        self.mem.close()

    def abandon(self) -> None:
        """Non-collective release for the recovery path (`SymmetricMemory.abandon`)."""
        self.mem.abandon()
