"""Harness of the per-pass compiler tests (the reference keeps one directory per pass under
nkigen/tests/passes/ with FileCheck-style IR assertions plus an execution check, nkigen/tests/harness.py:55-79).

`run_kernel_test(kernel, inputs, stop_after=..., check=...)` runs the native pipeline up to a pass and
  * matches `check`, a block of ``CHECK:`` / ``CHECK-NOT:`` / ``CHECK-COUNT-n:`` lines, against the IR text
    (CHECK lines must match in order, each as a substring of some later line; a CHECK-NOT must not occur
    between its neighbouring CHECK matches),
  * evaluates the IR after the pass with the NumPy interpreter and compares it with calling the kernel
    directly on NumPy arrays (direct mode), so every pass is also checked to preserve semantics.
"""
import re
from typing import Optional, Sequence

import numpy as np

from nkipy_b200.core.interp import evaluate
from nkipy_b200.core.ir import Graph
from nkipy_b200.nkigen import transforms as T


def filecheck(text: str, patterns: str) -> None:
    lines = text.splitlines()
    pos = 0
    pending_not = []
    for raw in patterns.strip().splitlines():
        raw = raw.strip()
        if not raw:
            continue
        m = re.match(r"CHECK(-NOT|-COUNT-(\d+))?:\s*(.*)", raw)
        if not m:
            raise ValueError(f"bad check line: {raw}")
        kind, count, pat = m.group(1), m.group(2), m.group(3)
        if kind == "-NOT":
            pending_not.append(pat)
            continue
        if kind and kind.startswith("-COUNT"):
            got = sum(pat in ln for ln in lines)
            assert got == int(count), f"expected {count} lines with {pat!r}, found {got}\n{text}"
            continue
        found = next((i for i in range(pos, len(lines)) if pat in lines[i]), None)
        assert found is not None, f"CHECK: {pat!r} not found after line {pos}\n{text}"
        for np_ in pending_not:
            assert not any(np_ in ln for ln in lines[pos:found]), f"CHECK-NOT: {np_!r} present\n{text}"
        pending_not = []
        pos = found + 1
    for np_ in pending_not:
        assert not any(np_ in ln for ln in lines[pos:]), f"CHECK-NOT: {np_!r} present\n{text}"


def ir_after(kernel_or_text, stop_after=None, passes: Optional[Sequence[str]] = None, **options) -> str:
    text = kernel_or_text if isinstance(kernel_or_text, str) else kernel_or_text.to_ir()
    if passes is not None:
        return T.apply_passes(text, list(passes), **options)
    return T.apply_complete_knob_pipeline(text, stop_after=stop_after, **options)


def run_kernel_test(kernel, inputs, stop_after=None, passes=None, check: str = "", rtol=1e-5, atol=1e-6,
                    **options) -> Graph:
    text = ir_after(kernel, stop_after=stop_after, passes=passes, **options)
    if check:
        filecheck(text, check)
    g = Graph.from_text(text)
    expected = kernel(*[np.array(a) for a in inputs])
    expected = list(expected) if isinstance(expected, (tuple, list)) else [expected]
    got = evaluate(g, list(inputs))
    assert len(got) == len(expected)
    for o, e in zip(got, expected):
        np.testing.assert_allclose(np.asarray(o, dtype=np.float64), np.asarray(e, dtype=np.float64), rtol=rtol,
                                   atol=atol)
    return g


def node(g: Graph, opcode: str, nth: int = 0):
    return [n for n in g.nodes if n.opcode == opcode][nth]
