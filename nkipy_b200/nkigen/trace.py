"""Standalone frontend of the native backend (nkigen/nkigen/trace.py:86-164 in the reference).

    @trace(input_specs=[((128, 256), "f32"), ((256, 64), "f32")])
    def kernel(a, b):
        return np.tanh(a @ b)

    ir_text = kernel.to_ir()              # (alias: to_mlir) IR text, inputs named in_tensor_{i}
    kernel(a, b)                          # direct mode on NumPy arrays
"""

from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np

from ..core.dtypes import dtype_from_name
from ..core.ir import Graph
from ..core.tensor import NKIPyTensorRef
from ..core.trace import NKIPyKernel

TracedArray = NKIPyTensorRef


class TracedKernel:
    def __init__(self, func: Callable, input_specs: Sequence[Tuple[Sequence[int], str]]):
        self.func = func
        self.input_specs = [(tuple(s), d) for s, d in input_specs]
        self._graph: Optional[Graph] = None
        self.__name__ = func.__name__

    def __call__(self, *args, **kwargs):
        return self.func(*args, **kwargs)

    def graph(self) -> Graph:
        if self._graph is None:
            args = [np.zeros(s, dtype=dtype_from_name(d) if isinstance(d, str) else d) for s, d in self.input_specs]
            g = NKIPyKernel(self.func, "nkigen").specialize(*args)
            self._graph = g
        return self._graph

    def to_ir(self) -> str:
        return self.graph().to_text()

    to_mlir = to_ir


def trace(func=None, *, input_specs: Optional[Sequence[Tuple[Sequence[int], str]]] = None):
    if input_specs is None:
        raise TypeError("trace needs input_specs=[(shape, dtype), ...]")

    def wrap(f):
        return TracedKernel(f, input_specs)

    return wrap(func) if func is not None else wrap
