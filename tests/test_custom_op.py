"""Hand-written CUDA kernels as operations of traced programs, on the CPU: the reference implementation runs in
direct mode and in the interpreter, the trace records source, launch geometry and the alias map, the code generator
emits the source and one launch per call (behaviours of the reference's tests/unit/test_nki.py: a kernel with a grid,
a simple one, one op called with two shapes, operand order, several outputs, mutable operands)."""
import shutil
import subprocess

import numpy as np
import pytest

from nkipy_b200.compiler.codegen import generate
from nkipy_b200.core.compile import trace
from nkipy_b200.core.cuda_op import CudaCustomOp, cuda_custom_op
from nkipy_b200.core.interp import evaluate
from utils import check, trace_kernel

AXPY = '''extern "C" __global__ void axpy_kernel(const float* x, const float* y, float* out, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = 2.f * x[i] + y[i];
}'''
R = np.random.default_rng(0)


def _axpy(n, **kw):
    return cuda_custom_op("axpy", AXPY, "axpy_kernel", [((n,), "f32")], grid=((n + 127) // 128,), block=(128,),
                          reference=lambda x, y: 2 * x + y, **kw)


def test_direct_mode_runs_the_reference():
    op = _axpy(64)
    x, y = R.standard_normal(64).astype(np.float32), R.standard_normal(64).astype(np.float32)
    np.testing.assert_allclose(op(x, y), 2 * x + y)
    with pytest.raises(NotImplementedError):
        cuda_custom_op("noref", AXPY, "axpy_kernel", [((4,), "f32")])(x[:4], y[:4])


def test_trace_records_source_geometry_and_result_types():
    op = _axpy(300)
    x = np.zeros(300, np.float32)
    g = trace(lambda a, b: op(a, b) * 0.5).specialize(x, x)
    (node,) = [n for n in g.nodes if n.opcode == "custom_call"]
    assert node.attrs["entry"] == "axpy_kernel" and node.attrs["source"] == AXPY
    assert node.attrs["grid"] == [3, 1, 1] and node.attrs["block"] == [128, 1, 1] and node.attrs["smem"] == 0
    assert node.attrs["result_types"] == [[[300], "f32"]]
    assert tuple(node.outputs[0].shape) == (300,)


def test_one_op_object_called_with_two_shapes_gives_two_calls():
    small, large = _axpy(32), _axpy(96)

    def kernel(a, b):
        return small(a[:32], b[:32]), large(a, b)

    a, b = R.standard_normal(96).astype(np.float32), R.standard_normal(96).astype(np.float32)
    g = trace(kernel).specialize(a, b)
    calls = [n for n in g.nodes if n.opcode == "custom_call"]
    assert [tuple(n.outputs[0].shape) for n in calls] == [(32,), (96,)]
    o0, o1 = evaluate(g, [a, b])
    np.testing.assert_allclose(o0, 2 * a[:32] + b[:32])
    np.testing.assert_allclose(o1, 2 * a + b)


def test_operands_keep_their_order():
    op = cuda_custom_op("sub", AXPY, "axpy_kernel", [((8,), "f32")], reference=lambda x, y: x - 3 * y)
    a, b = np.arange(8, dtype=np.float32), np.ones(8, np.float32)
    g = trace(lambda p, q: op(q, p)).specialize(a, b)            # swapped on purpose
    np.testing.assert_allclose(evaluate(g, [a, b])[0], b - 3 * a)
    (node,) = [n for n in g.nodes if n.opcode == "custom_call"]
    assert [i.id for i in node.inputs] == [g.params[1].id, g.params[0].id]


def test_several_outputs():
    op = cuda_custom_op("two", AXPY, "axpy_kernel", [((4, 4), "f32"), ((4,), "i32")],
                        reference=lambda x: (x * 2, x.sum(-1).astype(np.int32)))
    x = np.arange(16, dtype=np.float32).reshape(4, 4)
    g = trace(lambda a: op(a)).specialize(x)
    assert [o.dtype.name if hasattr(o.dtype, "name") else str(o.dtype) for o in g.outputs][1] in ("int32", "i32")
    o0, o1 = evaluate(g, [x])
    np.testing.assert_allclose(o0, x * 2)
    assert o1.tolist() == x.sum(-1).astype(np.int32).tolist()


def test_a_mutable_operand_becomes_an_aliased_output():
    op = _axpy(16, aliases={0: 0})
    x, y = np.arange(16, dtype=np.float32), np.ones(16, np.float32)

    def kernel(a, b):
        op(a, b)                       # writes its result over `a`

    direct = x.copy()
    kernel(direct, y)
    np.testing.assert_allclose(direct, 2 * x + y)              # direct mode updates the caller's array
    g = trace(kernel).specialize(x.copy(), y)
    assert [o.name for o in g.outputs] == ["a"] and g.aliases[0].param_name == "a"
    np.testing.assert_allclose(evaluate(g, [x.copy(), y])[0], 2 * x + y)


def test_builder_form_and_validation():
    def builder(input_specs, output_specs, factor):
        return AXPY.replace("2.f", f"{float(factor)}f")

    op = CudaCustomOp.from_kernel_builder(builder, name="scaled", entry="axpy_kernel", input_specs=[((8,), "f32")] * 2,
                                          output_specs=[((8,), "f32")], grid=(1,), block=(8,),
                                          reference=lambda x, y: 5 * x + y, factor=5)
    assert "5.0f" in op.source
    with pytest.raises(ValueError):
        cuda_custom_op("bad", AXPY, "axpy_kernel", [])
    with pytest.raises(Exception):
        cuda_custom_op("bad", AXPY, "axpy_kernel", [((4,), "float99")])


def test_generated_program_contains_the_source_and_compiles(tmp_path):
    op = _axpy(256)
    x = np.zeros(256, np.float32)
    prog = generate(trace(lambda a, b: op(a, b) + 1.0).specialize(x, x))
    assert AXPY.splitlines()[0] in prog.source
    assert any(l.kernel == "axpy_kernel" and tuple(l.grid) == (2, 1, 1) and tuple(l.block) == (128, 1, 1)
               for l in prog.launches)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if shutil.which(nvcc) is None:
        pytest.skip("nvcc not installed")
    src = tmp_path / "k.cu"
    src.write_text(prog.source)
    r = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-cubin", "-o",
                        str(tmp_path / "k.cubin"), str(src)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-1500:]


# ------------------------------------------------------------------ the cross-backend handle and the shape-pinned form
def _double_builder(input_specs, output_specs, factor=2.0):
    n = int(np.prod(input_specs[0][0]))
    return {"source": f'extern "C" __global__ void scale_kernel(const float* x, float* y) '
                      f'{{ int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < {n}) y[i] = {factor}f * x[i]; }}',
            "entry": "scale_kernel", "grid": ((n + 255) // 256,), "block": (256,)}


def test_handle_needs_a_kernel_or_a_builder_and_specs_for_the_builder():
    from nkipy_b200.core.nki_op import nki_custom_op

    with pytest.raises(ValueError, match="At least one"):
        nki_custom_op()
    with pytest.raises(ValueError, match="input_specs and output_specs"):
        nki_custom_op(kernel_builder=_double_builder)
    with pytest.raises(TypeError, match="nki_kernel must be"):
        nki_custom_op(nki_kernel=lambda x: x)
    with pytest.raises(TypeError, match="unknown argument"):
        nki_custom_op(kernel_builder=_double_builder, input_specs=[((8,), "f32")], output_specs=[((8,), "f32")], tile=4)
    with pytest.raises((ValueError, KeyError, TypeError)):
        nki_custom_op(kernel_builder=_double_builder, input_specs=[((8,), "f33")], output_specs=[((8,), "f32")])


def test_handle_without_a_reference_raises_on_numpy_arrays_and_traces_fine():
    from nkipy_b200.core.nki_op import nki_custom_op

    op = nki_custom_op(kernel_builder=_double_builder, input_specs=[((8,), "f32")], output_specs=[((8,), "f32")])
    with pytest.raises(RuntimeError, match="not supported on backend 'cpu'"):
        op(np.ones(8, np.float32))
    g = trace_kernel(lambda x: op(x), np.ones(8, np.float32))
    node = next(n for n in g.nodes if n.opcode == "custom_call")
    assert node.attrs["entry"] == "scale_kernel" and node.attrs["grid"] == [1, 1, 1] and node.attrs["block"] == [256, 1, 1]
    assert "2.0f * x[i]" in node.attrs["source"]


@pytest.mark.parametrize("backend", ["hlo", "nkigen"])
def test_handle_picks_the_form_the_backend_prefers_and_falls_back(backend):
    from nkipy_b200.core.nki_op import nki_custom_op
    from nkipy_b200.core.trace import NKIPyKernel

    written = cuda_custom_op(name="written", source=_double_builder([((8,), "f32")], None)["source"], entry="scale_kernel",
                             output_specs=[((8,), "f32")], reference=lambda x: 2 * x)
    both = nki_custom_op(nki_kernel=written, kernel_builder=_double_builder, input_specs=[((8,), "f32")],
                         output_specs=[((8,), "f32")], name="built", reference=lambda x: 2 * x)
    g = NKIPyKernel(lambda x: both(x), backend).specialize(np.ones(8, np.float32))
    g = getattr(g, "graph", g)
    target = next(n for n in g.nodes if n.opcode == "custom_call").attrs["target"]
    assert target == ("written" if backend == "hlo" else "built")
    only_written = nki_custom_op(nki_kernel=written)
    only_built = nki_custom_op(kernel_builder=_double_builder, input_specs=[((8,), "f32")], output_specs=[((8,), "f32")],
                               name="built")
    for op, want in ((only_written, "written"), (only_built, "built")):
        g = NKIPyKernel(lambda x: op(x), backend).specialize(np.ones(8, np.float32))
        g = getattr(g, "graph", g)
        assert next(n for n in g.nodes if n.opcode == "custom_call").attrs["target"] == want
    np.testing.assert_array_equal(both(np.ones(8, np.float32)), np.full(8, 2, np.float32))


def test_handle_checks_operands_against_its_specs():
    from nkipy_b200.core.nki_op import nki_custom_op

    op = nki_custom_op(kernel_builder=_double_builder, input_specs=[((8,), "f32")], output_specs=[((8,), "f32")],
                       reference=lambda x: 2 * x)
    with pytest.raises(ValueError, match="takes 1 operand"):
        op(np.ones(8, np.float32), np.ones(8, np.float32))
    with pytest.raises(ValueError, match="built for f32"):
        op(np.ones(9, np.float32))
    with pytest.raises(ValueError, match="built for f32"):
        op(np.ones(8, np.float16))
    with pytest.raises(ValueError, match="built for f32"):
        trace_kernel(lambda x: op(x), np.ones((2, 8), np.float32))


def test_builder_is_called_once_and_gets_its_keyword_arguments():
    from nkipy_b200.core.nki_op import nki_custom_op

    calls = []

    def builder(input_specs, output_specs, factor):
        calls.append(factor)
        return _double_builder(input_specs, output_specs, factor)

    op = nki_custom_op(kernel_builder=builder, input_specs=[((8,), "f32")], output_specs=[((8,), "f32")],
                       builder_kwargs={"factor": 3.0}, reference=lambda x: 3 * x)
    x = np.arange(8, dtype=np.float32)
    g = trace(lambda a: op(op(a))).specialize(x)
    assert calls == [3.0]
    assert sum(n.opcode == "custom_call" for n in g.nodes) == 2
    np.testing.assert_array_equal(evaluate(g, [x])[0], 9 * x)
    np.testing.assert_array_equal(op(op(x)), 9 * x)


def test_wrapped_kernel_is_pinned_to_its_example_operands():
    from nkipy_b200.core.nki_op import NKICustomOp, wrap_nki_kernel

    written = cuda_custom_op(name="written", source="", entry="k", output_specs=[((4, 4), "f32")], grid=(1,), block=(16,),
                             reference=lambda a, b: a + b)
    op = wrap_nki_kernel(written, [np.ones((4, 4), np.float32), np.ones((4, 4), np.float32)], grid=(2, 2))
    assert isinstance(op, NKICustomOp)
    assert op.config["grid"] == [2, 2] and op.config["block"] == [16] and op.config["input_specs"] == [((4, 4), "f32")] * 2
    assert written.grid == (1,)                                   # the wrapped kernel itself is left alone
    np.testing.assert_array_equal(op(np.ones((4, 4), np.float32), np.ones((4, 4), np.float32)), np.full((4, 4), 2.0))
    with pytest.raises(ValueError, match="operand 1"):
        op(np.ones((4, 4), np.float32), np.ones((4, 5), np.float32))
    with pytest.raises(TypeError):
        wrap_nki_kernel(lambda a: a, [np.ones(4, np.float32)])


def test_decorator_form_of_the_nkigen_front_end():
    from nkipy_b200.nkigen.custom_op import custom_op

    @custom_op(input_specs=[((8,), "f32")], output_specs=[((8,), "f32")], reference=lambda x: 2 * x)
    def scale_kernel(input_specs, output_specs):
        return _double_builder(input_specs, output_specs)["source"]

    x = np.arange(8, dtype=np.float32)
    g = trace(lambda a: scale_kernel(a) + 1.0).specialize(x)
    np.testing.assert_array_equal(evaluate(g, [x])[0], 2 * x + 1)
    np.testing.assert_array_equal(scale_kernel(x) + 1.0, 2 * x + 1)
    node = next(n for n in g.nodes if n.opcode == "custom_call")
    assert node.attrs["target"] == "scale_kernel" and node.attrs["entry"] == "scale_kernel"
