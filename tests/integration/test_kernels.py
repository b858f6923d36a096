"""Spec-driven integration test: every `kernel_specs` entry of tests/kernels/*.py runs on the default inputs of
its specification; direct mode (plain NumPy) is the oracle for the traced graph evaluated by the IR interpreter,
and for the compiled kernel on the device where there is one (the reference's counterpart:
tests/integration/test_kernels.py:56)."""
import copy
import glob
import importlib
import os

import numpy as np
import pytest

from nkipy_b200.core.specs import KernelSpec

from utils import check

HERE = os.path.dirname(os.path.abspath(__file__))


def collect_kernel_specs():
    found = {}
    for path in sorted(glob.glob(os.path.join(HERE, "..", "kernels", "*.py"))):
        stem = os.path.splitext(os.path.basename(path))[0]
        if stem == "__init__":
            continue
        module = importlib.import_module(f"kernels.{stem}")
        specs = getattr(module, "kernel_specs", None)
        if specs is None:
            continue
        for i, spec in enumerate(specs if isinstance(specs, list) else [specs]):
            found[f"{stem}:{i}:{getattr(spec.function, '__name__', 'kernel')}"] = spec
    return found


SPECS = collect_kernel_specs()


def test_specs_were_found():
    assert len(SPECS) >= 12
    assert all(isinstance(s, KernelSpec) and s.inputs for s in SPECS.values())


@pytest.mark.parametrize("name", sorted(SPECS))
def test_kernel_default(name):
    spec = SPECS[name]
    if not spec.is_pure_numpy:
        pytest.skip("not a pure NumPy kernel")
    inputs = spec.default_inputs(np.random.default_rng(0))
    for s, x in zip(spec.inputs, inputs):
        if hasattr(s, "shape_spec"):
            assert s.shape_spec.is_valid(np.shape(x)) and s.dtype_spec.is_valid(np.asarray(x).dtype)
    check(spec.function, *inputs, rtol=2e-3, atol=2e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(SPECS))
def test_kernel_default_on_device(name):
    from nkipy_b200.runtime import baremetal_run_traced_kernel

    spec = SPECS[name]
    inputs = spec.default_inputs(np.random.default_rng(0))
    expected = spec.function(*copy.deepcopy(inputs))
    got = baremetal_run_traced_kernel(spec.function, *copy.deepcopy(inputs))
    expected = expected if isinstance(expected, tuple) else (expected,)
    got = got if isinstance(got, tuple) else (got,)
    for e, g in zip(expected, got):
        np.testing.assert_allclose(np.asarray(g, np.float64), np.asarray(e, np.float64), rtol=1e-2, atol=1e-2)
