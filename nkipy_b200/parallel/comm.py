"""Tensor-parallel process group plumbing.

One process per GPU, launched by ``torchrun`` (``RANK`` / ``LOCAL_RANK`` /
``WORLD_SIZE`` / ``MASTER_*`` in the environment), exactly like the reference
examples bootstrap with ``torch.distributed.init_process_group``
(examples/models/qwen3/qwen3.py:461-467).  NCCL carries device tensors, a gloo
group (or the default group on CPU) carries Python objects.  `TPGroup` is the
handle the models use; with one rank every collective is a no-op.
"""

from __future__ import annotations

import datetime
import os
from typing import List, Optional

import torch
import torch.distributed as dist


class TPGroup:
    """A tensor-parallel group: rank / world size and the collectives the models need."""

    def __init__(self, rank: int = 0, world_size: int = 1, group=None, device: Optional[torch.device] = None):
        self.rank = rank
        self.world_size = world_size
        self.group = group
        self.device = device

    # ------------------------------------------------------------------ constructors
    @classmethod
    def single(cls, device=None) -> "TPGroup":
        return cls(0, 1, None, torch.device(device) if device is not None else None)

    @classmethod
    def from_env(cls, backend: Optional[str] = None, timeout_s: int = 600) -> "TPGroup":
        """Initialise ``torch.distributed`` from the torchrun environment (idempotent)."""
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        local = int(os.environ.get("LOCAL_RANK", str(rank)))
        use_cuda = torch.cuda.is_available()
        device = torch.device(f"cuda:{local}") if use_cuda else torch.device("cpu")
        if use_cuda:
            torch.cuda.set_device(device)
        if world == 1:
            return cls(0, 1, None, device)
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29531")
            if backend is None:
                backend = "nccl" if use_cuda else "gloo"
            kwargs = {}
            if backend == "nccl":
                kwargs["device_id"] = device
            dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                    timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
        return cls(rank, world, dist.group.WORLD, device)

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world_size > 1:
            dist.all_reduce(t, group=self.group)
        return t

    def all_gather(self, t: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Concatenate along a new leading rank dimension: returns [world, *t.shape]."""
        if out is None:
            out = torch.empty((self.world_size,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        if self.world_size == 1:
            out[0].copy_(t)
            return out
        dist.all_gather_into_tensor(out.view(-1), t.contiguous().view(-1), group=self.group)
        return out

    def reduce_scatter(self, t: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum over ranks and keep this rank's slice of dim 0."""
        if self.world_size == 1:
            return t
        if out is None:
            out = torch.empty((t.shape[0] // self.world_size,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.reduce_scatter_tensor(out, t, group=self.group)
        return out

    def broadcast_object(self, obj, src: int = 0):
        if self.world_size == 1:
            return obj
        box: List = [obj]
        dist.broadcast_object_list(box, src=src, group=self.group)
        return box[0]

    def all_gather_object(self, obj) -> list:
        if self.world_size == 1:
            return [obj]
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self.group)
        return out

    def barrier(self) -> None:
        if self.world_size > 1:
            dist.barrier(group=self.group)

    def max_over_ranks(self, value: float) -> float:
        """Max of a host scalar over the ranks (used for device-timed numbers)."""
        if self.world_size == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=self.device if self.device else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())
