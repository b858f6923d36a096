"""Tiling / placement / fusion hints of the native backend
(nkigen/nkigen/knob.py:44-240 in the reference).

    knob(x).tile_op(tile_size=[128, 256], reduction_tile=[64])
    knob(x).layout(mem_space="Shared", partition_dim=0, tile_size=[128, 64])
    knob.fuse(a, b, c)

Hints are recorded on the node that produces the tensor (attribute ``_knob``) and are
consumed by `infer-layout`, `knob-driven-tiling` and `knob-driven-fusion`.  Memory
spaces: Global, Shared, Tensor (TMEM), Register, Peer; the reference's Hbm / Sbuf / Psum /
SharedHbm are accepted as aliases.  Outside a trace the calls are no-ops.
"""

from __future__ import annotations

from typing import Optional, Sequence

from ..core.knob import MEM_SPACES
from ..core.tensor import NKIPyTensorRef


def _node_of(x):
    if isinstance(x, NKIPyTensorRef):
        return x.backend_tensor.producer
    return None


class _Knob:
    def __init__(self, tensor):
        self.tensor = tensor

    def _merge(self, **fields):
        node = _node_of(self.tensor)
        if node is None:
            return self
        cur = dict(node.attrs.get("_knob") or {})
        cur.update({k: v for k, v in fields.items() if v is not None})
        node.attrs["_knob"] = cur
        return self

    def tile_op(self, tile_size: Optional[Sequence[int]] = None, reduction_tile: Optional[Sequence[int]] = None):
        return self._merge(tile_size=list(tile_size) if tile_size is not None else None,
                           reduction_tile=list(reduction_tile) if reduction_tile is not None else None)

    def layout(self, mem_space: Optional[str] = None, partition_dim: Optional[int] = None,
               tile_size: Optional[Sequence[int]] = None):
        if mem_space is not None and mem_space not in MEM_SPACES:
            raise ValueError(f"unknown mem_space {mem_space!r}; expected one of {sorted(MEM_SPACES)}")
        return self._merge(mem_space=MEM_SPACES[mem_space] if mem_space else None, partition_dim=partition_dim,
                           tile_size=list(tile_size) if tile_size is not None else None)


class _KnobEntry:
    def __call__(self, tensor) -> _Knob:
        return _Knob(tensor)

    _next_group = 0

    def fuse(self, *tensors):
        """Ask for the producers of these tensors to land in one fused kernel."""
        gid = _KnobEntry._next_group
        _KnobEntry._next_group += 1
        for t in tensors:
            _Knob(t)._merge(fuse_group=gid)
        return tensors


knob = _KnobEntry()
