"""Structured loops for traced kernels (nkigen/nkigen/control_flow.py:12-163 in the reference, which emits
an `scf.for`).

``fori_loop(lo, hi, body, init)`` calls ``body(i, carry) -> carry`` for ``i`` in ``range(lo, hi, step)``.
Bounds are compile-time integers.

* In direct mode (NumPy arrays, no trace) it is that Python loop; ``i`` is a `LoopIndex` (an int).
* While tracing, the body is traced **once** into a nested graph with a symbolic index (a 0-d int32
  tensor) and becomes one ``loop`` node of the IR, so the size of the IR does not grow with the trip
  count.  The carry is a tensor or a tuple / list of tensors whose shapes and dtypes the body must
  preserve; tensors of the enclosing kernel that the body reads are captured automatically.
* A body that needs the index as a Python integer (static slice bounds, shapes, Python branching on
  ``i``) cannot be traced symbolically: the loop is then unrolled while tracing, as if written out
  (``unroll=True`` asks for that directly).
"""

from __future__ import annotations

from typing import Any, Callable, List

import numpy as np


class LoopIndex(int):
    """The induction variable of a direct-mode or unrolled loop: an int (affine arithmetic on it stays a
    Python int)."""


def _flatten(carry) -> List[Any]:
    return list(carry) if isinstance(carry, (tuple, list)) else [carry]


def _unflatten(like, values: List[Any]):
    if isinstance(like, tuple):
        return tuple(values)
    if isinstance(like, list):
        return list(values)
    return values[0]


def _unrolled(lower, upper, step, body, init):
    carry = init
    for i in range(lower, upper, step):
        carry = body(LoopIndex(i), carry)
    return carry


def fori_loop(lower: int, upper: int, body: Callable[[Any, Any], Any], init: Any, step: int = 1,
              unroll: bool = False):
    if not all(isinstance(v, (int, np.integer)) and not isinstance(v, bool) for v in (lower, upper, step)):
        raise TypeError("fori_loop bounds must be compile-time integers")
    lower, upper, step = int(lower), int(upper), int(step)
    if step <= 0:
        raise ValueError("fori_loop step must be positive")
    from ..core.backend import get_context

    ctx = get_context()
    if ctx is None or unroll or upper <= lower:
        return _unrolled(lower, upper, step, body, init)
    try:
        return _traced_loop(ctx, lower, upper, step, body, init)
    except _NeedsStaticIndex:
        return _unrolled(lower, upper, step, body, init)


class _NeedsStaticIndex(Exception):
    pass


def _traced_loop(ctx, lower, upper, step, body, init):
    from ..core.backend import tracing
    from ..core.backend.hlo import HLOTraceContext
    from ..core.ir import Graph
    from ..core.ops._ir_impls import as_value
    from ..core.tensor import NKIPyTensorRef

    outer: Graph = ctx.module
    flat_init = [as_value(v) for v in _flatten(init)]

    class BodyGraph(Graph):
        """Nested graph of the loop body: values of the enclosing graph that the body touches become
        extra parameters (captures)."""

        def __init__(self, name):
            super().__init__(name)
            self.own = set()
            self.captured = []          # [(outer value, inner parameter)]

        def _value(self, shape, dtype, name=""):
            v = super()._value(shape, dtype, name)
            self.own.add(id(v))
            return v

        def add_node(self, opcode, inputs, attrs=None):
            mapped = []
            for v in inputs:
                if id(v) in self.own:
                    mapped.append(v)
                    continue
                for ov, ip in self.captured:
                    if ov is v:
                        mapped.append(ip)
                        break
                else:
                    ip = self.add_parameter(v.shape, v.dtype, name=f"captured{len(self.captured)}")
                    self.captured.append((v, ip))
                    mapped.append(ip)
            return super().add_node(opcode, mapped, attrs)

    bg = BodyGraph(f"{outer.name}_loop_body")
    idx = bg.add_parameter((), np.int32, name="i")
    carried_params = [bg.add_parameter(v.shape, v.dtype, name=f"carry{k}") for k, v in enumerate(flat_init)]
    bctx = HLOTraceContext(bg)
    bctx.backend_name = ctx.backend_name
    for attr in ("honours_knobs", "knobs"):
        if hasattr(ctx, attr):
            setattr(bctx, attr, getattr(ctx, attr))
    carry_in = _unflatten(init, [NKIPyTensorRef(p) for p in carried_params])
    try:
        with tracing(bctx):
            result = body(NKIPyTensorRef(idx), carry_in)
            flat_out = [as_value(v) for v in _flatten(result)]
    except (TypeError, IndexError, ValueError, NotImplementedError) as e:
        # the body used the index where only a Python integer works (slice bounds, shapes, range(...))
        raise _NeedsStaticIndex(str(e)) from e
    if len(flat_out) != len(flat_init):
        raise ValueError("fori_loop body must return a carry of the same structure as init")
    for a, b in zip(flat_out, flat_init):
        if tuple(a.shape) != tuple(b.shape) or a.dtype != b.dtype:
            raise ValueError(f"fori_loop body changed a carried value from {b.type_str()} to {a.type_str()}")
    # a result that is a captured outer value (or the untouched carry) must be a value of the body graph
    outs = []
    for v in flat_out:
        if id(v) not in bg.own:
            v = bg.add_node("copy", [v], {})[0]
        outs.append(v)
    bg.set_results(outs, [f"carry{k}" for k in range(len(outs))])
    node_outs = outer.add_node("loop", flat_init + [ov for ov, _ in bg.captured],
                               {"lower": lower, "upper": upper, "step": step, "num_carried": len(flat_init),
                                "body": bg.to_text(with_locations=False)})
    return _unflatten(init, [NKIPyTensorRef(v) for v in node_outs])
