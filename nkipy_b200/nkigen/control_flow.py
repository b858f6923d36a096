"""Structured loops for traced kernels (nkigen/nkigen/control_flow.py:12-163 in the reference).

``fori_loop(lo, hi, body, init)`` calls ``body(i, carry) -> carry`` for ``i`` in
``range(lo, hi)``.  Bounds are compile-time integers; the loop is unrolled while tracing, so
``i`` is a plain Python int (`LoopIndex`) usable in slices and arithmetic.  In direct mode
it is the same Python loop over NumPy arrays.
"""

from __future__ import annotations

from typing import Any, Callable


class LoopIndex(int):
    """The induction variable: an int (affine arithmetic on it stays a Python int)."""


def fori_loop(lower: int, upper: int, body: Callable[[int, Any], Any], init: Any, step: int = 1):
    if not all(isinstance(v, int) for v in (lower, upper, step)):
        raise TypeError("fori_loop bounds must be compile-time integers")
    if step <= 0:
        raise ValueError("fori_loop step must be positive")
    carry = init
    for i in range(lower, upper, step):
        carry = body(LoopIndex(i), carry)
    return carry
