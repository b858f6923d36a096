"""Process-group layouts beyond one tensor-parallel group.

* data parallel: the world is split into `dp` independent replicas of `tp` ranks each (ranks
  [r * tp, (r + 1) * tp) form replica r); a replica serves its own requests, nothing is synchronised
  between replicas during inference.  `replica_groups(world, tp)` gives the same grouping in the
  list-of-lists form that the traced collectives take (nkipy/src/nkipy/core/ops/collectives.py:15-88).
* pipeline parallel: `PipelineStage` runs a contiguous slice of layers and passes the residual stream to
  the next stage with point-to-point send / recv (NCCL on GPUs, gloo on CPU ranks).  The reference has
  neither; both are thin host-side wrappers here.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .comm import TPGroup


def replica_groups(world_size: int, tp: int) -> List[List[int]]:
    if world_size % tp:
        raise ValueError("world size must be a multiple of the tensor-parallel size")
    return [list(range(r * tp, (r + 1) * tp)) for r in range(world_size // tp)]


def make_replica_group(tp_size: int, backend: Optional[str] = None) -> Tuple[TPGroup, int, int]:
    """Initialise torch.distributed from the environment and return (this rank's tensor-parallel group,
    replica index, number of replicas).  Every rank must call it (new_group is collective)."""
    world_tp = TPGroup.from_env(backend=backend)
    world, rank = world_tp.world_size, world_tp.rank
    if world == 1:
        return world_tp, 0, 1
    groups = replica_groups(world, tp_size)
    mine = None
    for ranks in groups:
        g = dist.new_group(ranks=ranks)
        if rank in ranks:
            mine = TPGroup(ranks.index(rank), tp_size, g, world_tp.device)
    return mine, rank // tp_size, len(groups)


class PipelineStage:
    """One pipeline stage: layers [first, last) of a model's layer list.

    `forward(x)` on stage 0 takes the embedded input; on later stages the input comes from the previous
    stage (pass None).  The last stage returns the output, earlier stages return None.  Micro-batches
    are pipelined by the caller issuing forward() per micro-batch: sends are asynchronous (`isend`), so a
    stage starts its next micro-batch while the previous one is still in flight to its successor."""

    def __init__(self, layer_fns, stage: int, num_stages: int, first_rank: int = 0, group=None):
        self.layer_fns, self.stage, self.num_stages = list(layer_fns), stage, num_stages
        self.prev = first_rank + stage - 1 if stage > 0 else None
        self.next = first_rank + stage + 1 if stage + 1 < num_stages else None
        self.group = group
        self._pending = []

    @staticmethod
    def partition(num_layers: int, num_stages: int) -> List[Tuple[int, int]]:
        base, rem = divmod(num_layers, num_stages)
        out, start = [], 0
        for s in range(num_stages):
            n = base + (1 if s < rem else 0)
            out.append((start, start + n))
            start += n
        return out

    def forward(self, x: Optional[torch.Tensor], shape=None, dtype=None, device=None) -> Optional[torch.Tensor]:
        if self.prev is not None:
            x = torch.empty(shape, dtype=dtype, device=device)
            dist.recv(x, src=self.prev, group=self.group)
        for f in self.layer_fns:
            x = f(x)
        if self.next is not None:
            self._pending = [w for w in self._pending if not w[0].is_completed()]
            self._pending.append((dist.isend(x, dst=self.next, group=self.group), x))   # keep x alive until sent
            return None
        return x

    def drain(self) -> None:
        for w, _ in self._pending:
            w.wait()
        self._pending = []
