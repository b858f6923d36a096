"""Trace-context plumbing shared by the frontend and the runtime.

Mirrors the surface of the reference's nkipy.core.backend
(nkipy/src/nkipy/core/backend/__init__.py:25-173): `TensorPlaceholder`, `AliasInfo`,
the `ComputationIR` protocol, `prepare_io_mapping`, the `tracing(ctx)` context
manager and `get_backend()` ("cpu" when nothing is being traced).  The active
context is kept per thread here.
"""

from __future__ import annotations

import threading
from contextlib import contextmanager
from typing import List, Optional, Protocol, Tuple, runtime_checkable

from ..ir import AliasInfo, TensorPlaceholder, prepare_io_mapping

__all__ = ["TensorPlaceholder", "AliasInfo", "ComputationIR", "prepare_io_mapping", "tracing", "get_backend",
           "get_context", "set_source_location"]

_state = threading.local()


@runtime_checkable
class ComputationIR(Protocol):
    """What the runtime needs from any traced program."""

    @property
    def inputs(self) -> List[TensorPlaceholder]: ...

    @property
    def outputs(self) -> List[TensorPlaceholder]: ...

    @property
    def aliases(self) -> List[AliasInfo]: ...

    @property
    def auto_aliased_indices(self) -> set: ...

    def content_hash(self, compiler_args: str) -> str: ...


@contextmanager
def tracing(ctx):
    """Activate `ctx` (an object with `backend_name` and `set_source_location`) for this thread."""
    prev = getattr(_state, "ctx", None)
    _state.ctx = ctx
    try:
        yield ctx
    finally:
        _state.ctx = prev


def get_context():
    return getattr(_state, "ctx", None)


def get_backend() -> str:
    ctx = get_context()
    return ctx.backend_name if ctx is not None else "cpu"


def set_source_location(location: Optional[Tuple[str, int]]) -> None:
    ctx = get_context()
    if ctx is not None:
        ctx.set_source_location(location)
