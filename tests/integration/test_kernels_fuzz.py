"""Fuzz test: ten random valid (shape, dtype) draws per kernel specification, direct mode against the interpreted
trace (the reference's counterpart: tests/integration/test_kernels_fuzz.py:75)."""
import numpy as np
import pytest

from utils import check
from .test_kernels import SPECS

FUZZ_ITERATIONS = 10


@pytest.mark.parametrize("name", sorted(SPECS))
def test_kernel_fuzz(name):
    spec = SPECS[name]
    if not spec.is_pure_numpy:
        pytest.skip("not a pure NumPy kernel")
    rng = np.random.default_rng(abs(hash(name)) % (2 ** 31))
    seen = set()
    for _ in range(FUZZ_ITERATIONS):
        inputs = spec.random_inputs(rng)
        for s, x in zip(spec.inputs, inputs):
            if hasattr(s, "shape_spec"):
                assert s.shape_spec.is_valid(np.shape(x)), (name, np.shape(x))
                assert s.dtype_spec.is_valid(np.asarray(x).dtype)
        seen.add(tuple((np.shape(x), str(np.asarray(x).dtype)) for x in inputs))
        half = any(np.asarray(x).dtype == np.float16 for x in inputs)
        check(spec.function, *inputs, rtol=2e-2 if half else 2e-3, atol=2e-2 if half else 2e-3)
    assert len(seen) >= 1
