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
