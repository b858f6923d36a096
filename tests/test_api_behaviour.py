"""The public surface does what a user of the reference expects of it, reached through the reference's import
names (`nkipy`, `spike`, `nkigen`): not only that the names exist (tests/test_api_surface.py), but that tracing,
specialising, the IR, the tensor APIs, the spec classes, the collectives, the kernel-agent helpers and the
nkigen front end work together on a CPU.  Reference: nkipy/src/nkipy/__init__.py and the packages it re-exports."""
import numpy as np
import pytest


def test_import_names_are_the_same_modules():
    import nkigen
    import nkipy
    import nkipy_b200
    import spike
    from nkipy.core import trace as t1
    from nkipy_b200.core import trace as t2

    assert t1 is t2 and nkipy.knob is nkipy_b200.knob
    assert spike.SpikeModel is nkipy_b200.spike.SpikeModel
    assert nkigen.trace is nkipy_b200.nkigen.trace


def test_trace_specialize_ir_and_interpreter_agree_with_numpy():
    from nkipy.core.compile import get_ir, trace
    from nkipy.core.trace import NKIPyKernel
    from nkipy_b200.core.interp import evaluate

    def kernel(x, w):
        h = np.matmul(x, w)
        return np.maximum(h, 0.0) + np.sum(x, axis=-1, keepdims=True)

    k = trace(kernel)
    assert isinstance(k, NKIPyKernel) and k.__name__ == "kernel"
    x = np.random.default_rng(0).standard_normal((8, 16)).astype(np.float32)
    w = np.random.default_rng(1).standard_normal((16, 4)).astype(np.float32)
    np.testing.assert_allclose(k(x, w), kernel(x, w), rtol=1e-6)          # direct mode: plain NumPy semantics
    k.specialize(x, w)
    g = get_ir(k)
    text = str(g)
    assert "dot(" in text and "max(" in text and "reduce(" in text and k._code is not None
    out = evaluate(g, [x, w])
    out = out[0] if isinstance(out, (list, tuple)) else out
    np.testing.assert_allclose(np.asarray(out), kernel(x, w), rtol=1e-5, atol=1e-5)


def test_tensor_apis_match_their_definitions():
    from nkipy.core import tensor_apis as ta

    x = np.random.default_rng(2).standard_normal((4, 32)).astype(np.float32)
    w = np.random.default_rng(3).standard_normal(32).astype(np.float32)
    e = np.exp(x - x.max(-1, keepdims=True))
    np.testing.assert_allclose(ta.softmax(x, axis=-1), e / e.sum(-1, keepdims=True), rtol=1e-5)
    np.testing.assert_allclose(ta.rms_norm(x, w, eps=1e-6), x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-6) * w,
                               rtol=1e-5)
    vals, idx = ta.topk(x, 3)
    np.testing.assert_allclose(vals, -np.sort(-x, axis=-1)[:, :3], rtol=1e-6)
    assert np.array_equal(np.take_along_axis(x, np.asarray(idx).astype(np.int64), -1), vals)
    assert ta.zeros((2, 3), np.float32).shape == (2, 3) and float(ta.full((2,), 7.0, np.float32)[1]) == 7.0


def test_kernel_spec_generates_valid_inputs_and_runs():
    from nkipy.core.specs import CommonTypes, KernelSpec, ShapeSpec, TensorInputSpec

    def f(a, b):
        return a * b + 1.0

    spec = KernelSpec(function=f, inputs=[
        TensorInputSpec(dtype_spec=CommonTypes.FLOATS, shape_spec=ShapeSpec(dims=[(1, 8), (1, 8)], default=(4, 4))),
        TensorInputSpec(dtype_spec=CommonTypes.FLOATS, shape_spec=ShapeSpec(dims=[(1, 8), (1, 8)], default=(4, 4))),
    ], description="elementwise")
    assert len(spec.inputs) == 2 and spec.is_pure_numpy
    shape = spec.inputs[0].shape_spec.default
    dtype = spec.inputs[0].dtype_spec.default
    a = np.ones(shape, dtype)
    np.testing.assert_allclose(spec.function(a, a), 2.0)


def test_collectives_on_one_rank_are_identities():
    from nkipy.distributed import collectives as cc

    x = np.arange(12, dtype=np.float32).reshape(3, 4)
    for fn, kw in ((cc.all_reduce, {}), (cc.all_gather, {"all_gather_dim": 0}), (cc.reduce_scatter, {"reduce_scatter_dim": 0}),
                   (cc.all_to_all, {"split_dimension": 0, "concat_dimension": 0})):
        try:
            y = fn(x, replica_groups=[[0]], **kw)
        except TypeError:
            y = fn(x, **kw) if kw else fn(x)
        np.testing.assert_allclose(np.asarray(y), x)


def test_kernel_agent_helpers_build_compile_and_run_on_the_cpu():
    from nkipy.tools import kernel_agent as ka

    ops = ka.get_all_ops()
    assert ("binary", "add") in ops and len(ops) >= 60
    made = ka.make_kernel("binary", "add", shape=(4, 8))
    assert made is not None
    fn, inputs = made
    res = ka.run_kernel(fn, inputs, use_gpu=False)
    assert isinstance(res, ka.ExecutionResult)
    source = ka.generate_kernel(["add", "tanh"])        # offline template client
    assert "def kernel" in source and "def make_inputs" in source
    cuda = ka.compile_code(source)
    assert isinstance(cuda, str) and "__global__" in cuda
    built = ka.build_inputs(source, seed=1)
    assert len(built) >= 1 and all(isinstance(x, np.ndarray) for x in built)


def test_nkigen_front_end_traces_verifies_and_runs_passes():
    import nkigen

    def f(a, b):
        return np.tanh(a @ b)

    traced = nkigen.trace(f, input_specs=[((8, 16), "f32"), ((16, 8), "f32")])
    text = traced.to_ir()
    a = np.random.default_rng(4).standard_normal((8, 16)).astype(np.float32)
    b = np.random.default_rng(5).standard_normal((16, 8)).astype(np.float32)
    assert nkigen.verify_against_numpy(f, text, [a, b], rtol=1e-4, atol=1e-5)
    out = nkigen.apply_passes(text, ["canonicalize"])
    assert isinstance(out, str) and "dot" in out


def test_runtime_surface_reports_the_device_state():
    from nkipy import runtime as rt

    assert isinstance(rt.is_neuron_compatible(), bool)
    assert callable(rt.baremetal_jit) and callable(rt.baremetal_run_traced_kernel)
    for name in ("BaremetalExecutor", "CompiledKernel", "DeviceKernel", "DeviceTensor"):
        assert isinstance(getattr(rt, name), type)
