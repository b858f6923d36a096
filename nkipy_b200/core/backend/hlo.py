"""The default trace backend ("hlo" in the reference's vocabulary).

The reference traces into an XLA HLO protobuf (nkipy/src/nkipy/core/backend/hlo.py);
here the same role is played by `nkipy_b200.core.ir.Graph`.  The reference's names
are kept as aliases so code written against that API keeps importing:
`HLOModule`, `HLOTensor`, `HLOTraceContext`, `get_hlo_context`,
`find_common_type_hlo`, `scalar_dtype_hlo`.
"""

from __future__ import annotations

from typing import Optional, Tuple

from ..dtypes import find_common_type, scalar_dtype
from ..ir import Graph, Node, Value
from . import get_context

HLOModule = Graph
HLOTensor = Value
HLOOp = Node
find_common_type_hlo = find_common_type
scalar_dtype_hlo = scalar_dtype


class HLOTraceContext:
    """Holds the graph under construction while a kernel function runs symbolically."""

    backend_name = "hlo"

    def __init__(self, module: Optional[Graph] = None):
        self.module = module if module is not None else Graph()

    @property
    def graph(self) -> Graph:
        return self.module

    def set_source_location(self, location: Optional[Tuple[str, int]]) -> None:
        self.module.set_source_location(location)

    def build_op(self, opcode: str, inputs, attrs=None):
        return self.module.add_node(opcode, inputs, attrs or {})


def get_hlo_context() -> HLOTraceContext:
    ctx = get_context()
    if ctx is None or ctx.backend_name not in ("hlo", "nkigen"):      # both trace the same tensor IR
        raise RuntimeError("no IR trace context is active")
    return ctx
