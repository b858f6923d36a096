"""Mixture-of-experts FFN block with expert parallelism.

The reference keeps every expert on every rank and shards the expert intermediate
dimension (tensor parallelism), evaluating experts with per-token loops or batched
gathers (examples/models/qwen3/kernels/transformer_layer.py:70-115,
examples/models/gpt_oss/kernels/feedforward.py:39-206).  Here the default is expert
parallelism: rank r owns experts [r * E / ep, (r + 1) * E / ep); activations are
replicated by the preceding tensor-parallel reduction, so *dispatch* is a local
sort-and-gather of the pairs routed to local experts, the experts run as two grouped
tcgen05 GEMMs (SwiGLU fused into the first), and *combine* sums the weighted expert
outputs per token locally and then over ranks.  `moe_parallel="tp"` reproduces the
reference's sharding with the same code path (all experts local, narrower experts).
"""

from __future__ import annotations

import torch

from .. import ops
from ..parallel.comm import TPGroup
from .config import ModelConfig


class MoEBlock:
    def __init__(self, cfg: ModelConfig, tp: TPGroup, moe_parallel: str = "ep"):
        self.cfg, self.tp, self.mode = cfg, tp, moe_parallel
        if moe_parallel == "ep" and cfg.num_experts % tp.world_size:
            raise ValueError("expert parallelism needs num_experts divisible by the number of ranks")
        self.num_local = cfg.num_experts // tp.world_size if moe_parallel == "ep" else cfg.num_experts
        self.expert_lo = tp.rank * self.num_local if moe_parallel == "ep" else 0

    def route(self, lw, x: torch.Tensor):
        # one 128-row weight tile: split the contraction so several SMs share the work
        logits = ops.linear(x, lw.router, splits=max(2, min(16, x.shape[1] // 256)))
        return ops.router_topk(logits, self.cfg.top_k, self.cfg.router_mode, bias=lw.router_bias)

    def _experts(self, lw, x: torch.Tensor):
        """Route, dispatch and run the local experts; returns (y_sorted, plan, routing weights)."""
        cfg = self.cfg
        T = x.shape[0]
        weights, experts = self.route(lw, x)
        plan = ops.moe_dispatch(x, experts, self.expert_lo, self.num_local)
        h = ops.grouped_linear(plan.x_sorted, lw.gate_up, plan.offsets, max_rows_per_group=T, gated=True,
                               bias=lw.gate_up_bias, act_limit=cfg.swiglu_limit, act_alpha=cfg.swiglu_alpha,
                               tiles=plan.tiles)
        y_sorted = ops.grouped_linear(h, lw.down, plan.offsets, max_rows_per_group=T, bias=lw.down_bias,
                                      tiles=plan.tiles)
        return y_sorted, plan, weights

    def forward(self, lw, x: torch.Tensor) -> torch.Tensor:
        """x [T, H] (normed hidden states, replicated over ranks) -> MoE output [T, H], summed over ranks."""
        y_sorted, plan, weights = self._experts(lw, x)
        y = ops.moe_combine(y_sorted, plan.pair_pos, weights, x.shape[0])
        self.tp.all_reduce(y)
        return y

    def forward_add_rmsnorm(self, lw, x: torch.Tensor, resid: torch.Tensor, next_norm: torch.Tensor):
        """MoE block + residual + next RMSNorm; returns (new residual, normed).  With the fused
        tensor-parallel runtime the combine kernel pushes its partial rows straight into the peers'
        buffers and the reducing norm kernel sums them (no library collective)."""
        cfg = self.cfg
        fused = getattr(self.tp, "fused", None)
        T = x.shape[0]
        if fused is not None and T <= fused.max_tokens:
            y_sorted, plan, weights = self._experts(lw, x)
            return fused.moe_combine_allreduce_add_rmsnorm(y_sorted, plan.pair_pos, weights, T, resid, next_norm,
                                                           cfg.rms_eps)
        y = self.forward(lw, x)
        return ops.add_rmsnorm(y, next_norm, residual_in=resid, eps=cfg.rms_eps)

    def forward_sharded(self, lw, x_local: torch.Tensor) -> torch.Tensor:
        """Expert-parallel block for tokens that are sharded over the ranks (x_local [T / ranks, H], this rank's
        slab): the rows travel to their experts' owners and back through peer memory
        (`parallel.moe_a2a.MoEAllToAll`).  Returns this rank's slab of the block output."""
        from ..parallel.moe_a2a import MoEAllToAll

        cfg = self.cfg
        T = x_local.shape[0]
        a2a = getattr(self, "_a2a", None)
        if a2a is None or a2a.max_local_tokens < T:
            if a2a is not None:
                a2a.close()
            cap = max(2048, 1 << (T - 1).bit_length())
            a2a = self._a2a = MoEAllToAll(self.tp, cap, cfg.top_k, cfg.hidden_size, cfg.num_experts)
        weights, experts = self.route(lw, x_local)
        return a2a.forward(x_local, experts, weights, lw.gate_up, lw.down, gate_up_bias=lw.gate_up_bias,
                           down_bias=lw.down_bias, act_limit=cfg.swiglu_limit, act_alpha=cfg.swiglu_alpha)
