"""Shared helpers of the frontend tests: direct mode is the oracle, the traced graph is
checked through the NumPy IR interpreter (after a text round trip)."""
import copy

import numpy as np

from nkipy_b200.core.interp import evaluate
from nkipy_b200.core.ir import Graph
from nkipy_b200.core.trace import NKIPyKernel

CPU_TOL = dict(rtol=1e-4, atol=1e-4)


def trace_kernel(fn, *args, **kwargs) -> Graph:
    k = NKIPyKernel(fn, "hlo")
    g = k.specialize(*args, **kwargs)
    g2 = Graph.from_text(g.to_text())
    assert g2.to_text(with_locations=False) == g.to_text(with_locations=False)
    return g2


def run_traced(fn, *args, **kwargs):
    g = trace_kernel(fn, *copy.deepcopy(args), **copy.deepcopy(kwargs))
    arrays = [a for a in args if isinstance(a, np.ndarray)] + [v for v in kwargs.values() if isinstance(v, np.ndarray)]
    from nkipy_b200.core.dtypes import sanitize_dtype

    arrays = [a.astype(sanitize_dtype(a.dtype)) for a in arrays]
    return g, evaluate(g, arrays)


def check(fn, *args, rtol=1e-4, atol=1e-4, **kwargs):
    """Direct-mode result of fn(*args) must equal the interpreted trace."""
    expected = fn(*copy.deepcopy(args), **copy.deepcopy(kwargs))
    g, got = run_traced(fn, *args, **kwargs)
    if expected is None:
        expected = []
    if not isinstance(expected, (tuple, list)):
        expected = [expected]
    user = [o for i, o in enumerate(got) if i not in g.auto_aliased_indices]
    assert len(user) == len(expected), (len(user), len(expected))
    for e, o in zip(expected, user):
        e = np.asarray(e)
        assert tuple(o.shape) == tuple(e.shape), (o.shape, e.shape)
        if e.dtype == np.bool_:
            e = e.astype(np.uint8)
        np.testing.assert_allclose(o.astype(np.float64), e.astype(np.float64), rtol=rtol, atol=atol)
    return g
