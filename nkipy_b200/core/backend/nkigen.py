"""Adapter names of the "nkigen" backend (nkipy/src/nkipy/core/backend/nkigen.py:24-180 in the
reference wraps an MLIR builder).  Here the nkigen backend traces the same tensor IR as the default
one; what differs is that knob annotations are honoured, parameters / results follow the
``in_tensor_{i}`` / ``output`` naming, and compilation is routed through the native pass pipeline.
These classes give code written against the reference's module the objects it expects."""

from __future__ import annotations

from typing import Optional

from ..ir import Graph, Value
from . import get_context
from .hlo import HLOTraceContext

NkiGenTensor = Value


class NkiGenTraceContext(HLOTraceContext):
    """Trace context whose knobs are kept (`honours_knobs`) for the native compiler."""

    backend_name = "nkigen"

    def __init__(self, module: Optional[Graph] = None):
        super().__init__(module)
        self.honours_knobs = True
        self.knobs = {}


class NkiGenIR:
    """`ComputationIR` view of a traced graph for the nkigen route: same inputs / outputs / aliases,
    content hash over the IR text (the reference hashes the MLIR text, backend/nkigen.py:174-179)."""

    def __init__(self, graph: Graph):
        self.graph = graph

    @property
    def inputs(self):
        return self.graph.inputs

    @property
    def outputs(self):
        return self.graph.outputs

    @property
    def aliases(self):
        return self.graph.aliases

    @property
    def auto_aliased_indices(self):
        return self.graph.auto_aliased_indices

    def content_hash(self, compiler_args: str = "") -> str:
        return self.graph.content_hash(compiler_args)

    def to_text(self) -> str:
        return self.graph.to_text()


def get_nkigen_context() -> NkiGenTraceContext:
    ctx = get_context()
    if ctx is None or not getattr(ctx, "honours_knobs", False):
        raise RuntimeError("no nkigen trace context is active")
    return ctx
