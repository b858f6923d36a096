"""Kernel wrapper and tracer.

`NKIPyKernel(func, backend)` wraps a plain NumPy function.  `specialize(*args)` runs
it once symbolically: every `np.ndarray` argument becomes a graph parameter wrapped
in an `NKIPyTensorRef`, every other argument stays a Python constant ("comptime"),
and the operations the function performs are recorded into a `Graph`.  Mutated
parameters (``x[...] = v`` / ``np.put_along_axis``) are appended as outputs aliased
to their input; outputs are named ``output{i}`` or, for aliased ones, after the
parameter; an aliased input is exposed as ``"<name>.must_alias_input"``; returning an
untouched parameter inserts a copy.  Same contract as the reference tracer
(nkipy/src/nkipy/core/trace.py:87-381).  Backends: "hlo" (alias "b200") traces into
this package's IR, "nkigen" traces the same IR and routes compilation through the
native pass pipeline, "cpu" needs no specialization.
"""

from __future__ import annotations

import inspect
import warnings
from typing import Any, Dict, List, Optional

import numpy as np

from ._numpy_dispatch import register_all_numpy_apis
from .backend import tracing
from .backend.hlo import HLOTraceContext
from .dtypes import sanitize_array
from .ir import AliasInfo, Graph
from .tensor import NKIPyTensorRef

register_all_numpy_apis()

_BACKENDS = ("hlo", "b200", "nkigen", "cpu")


def _convert_args(sig, bound, convert):
    args, kwargs = [], {}
    for name, arg in bound.arguments.items():
        p = sig.parameters[name]
        if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD):
            args.append(convert(name, arg))
        elif p.kind == p.KEYWORD_ONLY:
            kwargs[name] = convert(name, arg)
        elif p.kind == p.VAR_POSITIONAL:
            args.extend(convert(f"{name}_{i}", a) for i, a in enumerate(arg))
        else:
            kwargs.update({k: convert(k, v) for k, v in arg.items()})
    return args, kwargs


class NKIPyKernel:
    """A NumPy function that can run directly on arrays or be traced into the IR."""

    def __init__(self, func, backend: str = "hlo"):
        if backend not in _BACKENDS:
            raise ValueError(f"Unknown backend {backend}")
        self.func = func
        self.backend = backend
        self._code: Optional[Graph] = None
        self._params: List[NKIPyTensorRef] = []

    @property
    def __name__(self):
        return self.func.__name__

    def __repr__(self):
        return f"<NKIPyKernel '{self.func.__name__}' backend='{self.backend}'>"

    def __call__(self, *args, **kwargs):
        """CPU direct mode: just run the NumPy function."""
        return self.func(*args, **kwargs)

    @classmethod
    def trace(cls, func=None, *, backend: str = "hlo"):
        """Decorator form: ``@NKIPyKernel.trace`` or ``@NKIPyKernel.trace(backend=...)``."""
        if func is None:
            return lambda f: cls(f, backend)
        return cls(func, backend)

    # ------------------------------------------------------------------ specialization
    def specialize(self, *args, **kwargs):
        if self.backend == "cpu":
            warnings.warn("CPU backend does not require specialization", stacklevel=2)
            return None
        sig = inspect.signature(self.func)
        bound = sig.bind(*args, **kwargs)
        bound.apply_defaults()
        graph = Graph(self.func.__name__)
        ctx = HLOTraceContext(graph)
        ctx.backend_name = "nkigen" if self.backend == "nkigen" else "hlo"      # what get_backend() reports meanwhile
        if self.backend == "nkigen":
            ctx.honours_knobs = True
            ctx.knobs = {}
        params: List[NKIPyTensorRef] = []

        def convert(name: str, arg: Any):
            if isinstance(arg, NKIPyTensorRef):
                raise TypeError("kernels are specialized with concrete arrays, not traced tensors")
            if isinstance(arg, np.ndarray):
                arr = sanitize_array(arg, name)
                v = graph.add_parameter(arr.shape, arr.dtype, name=name)
                ref = NKIPyTensorRef(v, name=name, original_parameter=v)
                params.append(ref)
                return ref
            return arg

        with tracing(ctx):
            cargs, ckwargs = _convert_args(sig, bound, convert)
            result = self.func(*cargs, **ckwargs)
            self._finish(graph, params, result)
        if self.backend == "nkigen":
            self._apply_nkigen_conventions(graph, ctx)
        self._code = graph
        self._params = params
        return graph

    @staticmethod
    def _apply_nkigen_conventions(graph: Graph, ctx) -> None:
        for vid, hint in ctx.knobs.items():
            for n in graph.nodes:
                if any(o.id == vid for o in n.outputs):
                    cur = dict(n.attrs.get("_knob") or {})
                    cur.update({k: v for k, v in hint.items() if v is not None})
                    n.attrs["_knob"] = cur
        _nkigen_names(graph)

    def _finish(self, graph: Graph, params: List[NKIPyTensorRef], result) -> None:
        from . import ops

        if result is None:
            returned: List[Any] = []
        elif isinstance(result, (tuple, list)):
            returned = list(result)
        else:
            returned = [result]
        values, names, aliases = [], [], []
        param_index = {id(p): i for i, p in enumerate(params)}
        seen_mutated = set()
        for out in returned:
            if not isinstance(out, NKIPyTensorRef):
                out = ops.constant(np.asarray(out))
            pi = param_index.get(id(out))
            idx = len(values)
            if pi is not None and params[pi]._is_mutated:
                values.append(out.backend_tensor)
                names.append(params[pi]._name)
                aliases.append(AliasInfo(idx, pi, params[pi]._name, True))
                seen_mutated.add(pi)
            elif pi is not None or out.backend_tensor in graph.params or out.backend_tensor in values:
                # an untouched parameter (or a value returned twice) needs a buffer of its own
                values.append(graph.op("copy", out.backend_tensor))
                names.append(f"output{idx}")
            else:
                values.append(out.backend_tensor)
                names.append(f"output{idx}")
        for pi, p in enumerate(params):
            if p._is_mutated and pi not in seen_mutated:
                idx = len(values)
                values.append(p.backend_tensor)
                names.append(p._name)
                aliases.append(AliasInfo(idx, pi, p._name, False))
        for a in aliases:
            graph.params[a.param_index].name = f"{a.param_name}.must_alias_input"
        graph.set_results(values, names, aliases)


def _nkigen_names(graph: Graph) -> None:
    """Inputs are called in_tensor_{i}, outputs `output` / `output_{i}` on the native backend
    (aliased outputs keep the parameter name)."""
    aliased_out = {a.output_index for a in graph.alias_list}
    aliased_in = {a.param_index for a in graph.alias_list}
    for i, p in enumerate(graph.params):
        if i not in aliased_in:
            p.name = f"in_tensor_{i}"
    free = [i for i in range(len(graph.results)) if i not in aliased_out]
    for k, i in enumerate(free):
        graph.result_names[i] = "output" if len(free) == 1 else f"output_{k}"


def trace(func=None, *, backend: str = "hlo"):
    """``trace(fn)`` / ``@trace`` / ``@trace(backend="cpu")`` -> `NKIPyKernel`."""
    return NKIPyKernel.trace(func, backend=backend)
