"""Tiling / placement hint (nkipy/src/nkipy/core/knob.py:17-70 in the reference).

``knob(tensor, partition_dim=, mem_space=, tile_size=, reduction_tile=)`` attaches a hint
to the value a traced tensor denotes.  The native pass pipeline ("nkigen" backend) reads
it (tile shape, memory space Global / Shared / Tensor / Register; the reference's names
Hbm / Sbuf / Psum / SharedHbm are accepted as aliases); the default backend warns that the
hint has no effect there; in CPU direct mode it is a no-op.  Returns the tensor.
"""

from __future__ import annotations

import warnings
from typing import Optional, Sequence

from .backend import get_backend, get_context

MEM_SPACES = {"Global": "Global", "Shared": "Shared", "Tensor": "Tensor", "Register": "Register", "Peer": "Peer",
              "Hbm": "Global", "Sbuf": "Shared", "Psum": "Tensor", "SharedHbm": "Global", "Constant": "Global"}


def knob(tensor, partition_dim: Optional[int] = None, mem_space: Optional[str] = None,
         tile_size: Optional[Sequence[int]] = None, reduction_tile: Optional[Sequence[int]] = None):
    backend = get_backend()
    if backend == "cpu":
        return tensor
    if mem_space is not None and mem_space not in MEM_SPACES:
        raise ValueError(f"unknown mem_space {mem_space!r}; expected one of {sorted(MEM_SPACES)}")
    ctx = get_context()
    hints = getattr(ctx, "knobs", None)
    if hints is None or not getattr(ctx, "honours_knobs", False):
        warnings.warn("knob() is only effective with backend='nkigen' (the native pass pipeline); ignored here", stacklevel=2)
        return tensor
    hints[tensor.backend_tensor.id] = {
        "partition_dim": partition_dim, "mem_space": MEM_SPACES.get(mem_space) if mem_space else None,
        "tile_size": list(tile_size) if tile_size is not None else None,
        "reduction_tile": list(reduction_tile) if reduction_tile is not None else None,
    }
    return tensor
