"""CPU execution oracle for IR at any pipeline stage (the role of the reference's LLVM-JIT
path, nkigen/nkigen/llvm.py and nkigen/nkigen/execution.py): the IR text is parsed and
evaluated with the NumPy interpreter, so the result after any `stop_after` can be compared
with the untransformed program or with the NumPy function itself."""

from __future__ import annotations

from typing import Callable, List, Sequence

import numpy as np

from ..core.interp import evaluate
from ..core.ir import Graph


def run_ir(ir_text: str, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
    return evaluate(Graph.from_text(ir_text), list(inputs))


def verify_against_numpy(func: Callable, ir_text: str, inputs: Sequence[np.ndarray], rtol: float = 1e-5,
                         atol: float = 1e-8) -> bool:
    """Raises AssertionError when the IR's result differs from func(*inputs)."""
    expected = func(*[np.array(a) for a in inputs])
    expected = list(expected) if isinstance(expected, (tuple, list)) else [expected]
    got = run_ir(ir_text, inputs)
    assert len(got) >= len(expected), (len(got), len(expected))
    for e, g in zip(expected, got):
        np.testing.assert_allclose(np.asarray(g, dtype=np.float64), np.asarray(e, dtype=np.float64), rtol=rtol,
                                   atol=atol)
    return True
