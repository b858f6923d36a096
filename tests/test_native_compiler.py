"""Native C++ pass pipeline: every pass preserves semantics (checked with the NumPy IR
interpreter), the opt driver honours stop_after / dump_dir, knobs reach the annotations."""
import os
import subprocess

import numpy as np
import pytest

from nkipy_b200 import nkigen
from nkipy_b200.compiler.native import build, opt_path
from nkipy_b200.core.interp import evaluate
from nkipy_b200.core.ir import Graph
from nkipy_b200.nkigen import transforms as T
from utils import trace_kernel

build()
R = np.random.default_rng(0)


def f32(*s):
    return R.standard_normal(s).astype(np.float32)


def attention(q, k, v):
    s = (q @ np.transpose(k, (1, 0))) / np.sqrt(np.float32(q.shape[-1]))
    s = s + np.zeros_like(s)
    p = np.exp(s - np.max(s, axis=-1, keepdims=True))
    p = p / np.sum(p, axis=-1, keepdims=True)
    return (p @ v) * 1.0 + (p @ v) ** 2


def _graph():
    q, k, v = f32(64, 32), f32(48, 32), f32(48, 16)
    return trace_kernel(attention, q, k, v), [q, k, v]


def test_every_pass_preserves_semantics():
    g, ins = _graph()
    base = evaluate(g, ins)[0]
    text = g.to_text()
    for name in [p for p in T.pass_list() if not p.startswith("py:")]:
        text = T.apply_passes(text, [name])
        out = evaluate(Graph.from_text(text), ins)[0]
        np.testing.assert_allclose(out, base, rtol=1e-5, atol=1e-6, err_msg=f"after {name}")
    final = Graph.from_text(text)
    ops = [n.opcode for n in final.nodes]
    assert len(final.nodes) < len(g.nodes)                        # zero fill / x*1 / transpose were folded
    assert "pow" not in ops and "transpose" not in ops
    dots = [n for n in final.nodes if n.opcode == "dot"]
    assert dots[0].attrs["rhs_contract"] == [1] and dots[0].attrs["_b_major"] == "K"
    assert all("_tile" in d.attrs and "_tiling" in d.attrs and "_stages" in d.attrs and d.attrs["_path"] == "simt"
               for d in dots)
    assert any("_fuse_group" in n.attrs for n in final.nodes) and any("_buffer" in n.attrs for n in final.nodes)
    assert any("_last_use_of" in n.attrs for n in final.nodes)


def test_pipeline_stop_after_and_dump(tmp_path):
    g, ins = _graph()
    text = g.to_text()
    full = T.apply_complete_knob_pipeline(text, dump_dir=str(tmp_path / "d"))
    dumps = sorted(os.listdir(tmp_path / "d"))
    native = [p for p in T.pass_list() if not p.startswith("py:")]
    assert len(dumps) == len(native) and dumps[0] == "01_remove-redundant-zero-fill.ir"
    assert dumps[-1].startswith(f"{len(native):02d}_")
    by_name = T.apply_complete_knob_pipeline(text, stop_after="simplify-linalg")
    by_index = T.apply_complete_knob_pipeline(text, stop_after=6)
    assert by_name == by_index and "_tile" not in by_name
    by_group = T.apply_complete_knob_pipeline(text, stop_after="canonicalize")
    assert "_op_id" not in by_group and "_tile" not in by_group
    layout = T.apply_complete_knob_pipeline(text, stop_after="layout")
    assert "_tiling" in layout and "_buffer" not in layout
    ir, src = T.apply_complete_knob_pipeline(text, emit_cuda=True, dump_dir=str(tmp_path / "e"))
    assert 'extern "C" __global__' in src and any(f.endswith("_py_ir-to-cuda.cu") for f in os.listdir(tmp_path / "e"))
    np.testing.assert_allclose(evaluate(Graph.from_text(full), ins)[0], evaluate(g, ins)[0], rtol=1e-5, atol=1e-6)
    with pytest.raises(RuntimeError) as ei:
        T.apply_complete_knob_pipeline(text, stop_after="no-such-pass")
    assert "nkipy-b200-opt" in str(ei.value) and "stderr" in str(ei.value)


def test_opt_cli_and_errors(tmp_path):
    g, _ = _graph()
    src = tmp_path / "in.ir"
    src.write_text(g.to_text())
    out = subprocess.run([str(opt_path()), "--pass", "cse", "--pass", "canonicalize", str(src)], capture_output=True,
                         text=True)
    assert out.returncode == 0 and out.stdout.startswith("graph @attention")
    lst = subprocess.run([str(opt_path()), "--list-passes"], capture_output=True, text=True).stdout
    assert "insert-spill-reload" in lst and "legalize-layout" in lst and len(lst.strip().splitlines()) >= 22
    bad = subprocess.run([str(opt_path()), "--pass", "nope", str(src)], capture_output=True, text=True)
    assert bad.returncode == 1 and "unknown pass" in bad.stderr
    broken = subprocess.run([str(opt_path())], input="graph @k {\n  %1 = exp(%0) {} : f32[2]\n  return %1 {\"name\": \"o\"}\n}\n",
                            capture_output=True, text=True)
    assert broken.returncode == 1 and "undefined value" in broken.stderr
    with pytest.raises(RuntimeError):
        T.apply_passes(g.to_text(), ["nope"])


def test_knobs_tiles_and_budget():
    import ml_dtypes

    bf = ml_dtypes.bfloat16

    @nkigen.trace(input_specs=[((512, 1024), "bf16"), ((1024, 768), "bf16")])
    def mm(a, b):
        c = a @ b
        nkigen.knob(c).tile_op(tile_size=[128, 128], reduction_tile=[64])
        d = np.tanh(c)
        nkigen.knob(d).layout(mem_space="Sbuf")
        return d

    g = mm.graph()
    assert [p.name for p in g.inputs] == ["in_tensor_0", "in_tensor_1"] and g.outputs[0].name == "output"
    text = T.apply_complete_knob_pipeline(mm.to_ir())
    final = Graph.from_text(text)
    dot = next(n for n in final.nodes if n.opcode == "dot")
    assert dot.attrs["_tile"] == [128, 128, 64] and dot.attrs["_path"] == "tcgen05"
    assert dot.attrs["_tma_box_b"] == [64, 128] and dot.attrs["_mem"] == "Tensor" and "_knob" not in dot.attrs
    tanh = next(n for n in final.nodes if n.opcode == "tanh")
    assert tanh.attrs["_epilogue_of"] == dot.attrs["_op_id"]
    # a tiny shared-memory budget forces fewer stages, then smaller tiles, then an error
    small = Graph.from_text(T.apply_complete_knob_pipeline(mm.to_ir(), smem_capacity=70000))
    sd = next(n for n in small.nodes if n.opcode == "dot")
    assert sd.attrs["_stages"] < dot.attrs["_stages"] and sd.attrs["_smem_bytes"] <= 70000
    with pytest.raises(RuntimeError) as ei:
        T.apply_complete_knob_pipeline(mm.to_ir(), smem_capacity=20000)
    assert "insert-spill-reload" in str(ei.value)
    with pytest.raises(ValueError):
        nkigen.knob(np.zeros(2)).layout(mem_space="Nowhere")
    a = np.ones((4, 4), np.float32)
    assert nkigen.verify_against_numpy(lambda x: np.exp(x) * 2, nkigen.trace(lambda x: np.exp(x) * 2, input_specs=[((4, 4), "f32")]).to_ir(), [a])


def test_fori_loop_and_backend_knob_dispatch():
    from nkipy_b200 import knob as core_knob
    from nkipy_b200.core.trace import NKIPyKernel

    def scan(x):
        def body(i, acc):
            return acc + x[i] * (i + 1)

        return nkigen.fori_loop(0, 4, body, np.zeros(3, np.float32))

    x = f32(4, 3)
    g = trace_kernel(scan, x)
    np.testing.assert_allclose(evaluate(g, [x])[0], scan(x), rtol=1e-6)
    with pytest.raises(TypeError):
        nkigen.fori_loop(0, 2.5, lambda i, c: c, 0)

    def hinted(a):
        b = a * 2
        core_knob(b, partition_dim=0, mem_space="Sbuf", tile_size=[64, 32])
        return b

    assert hinted(x) is not None                                            # cpu: no-op
    with pytest.warns(UserWarning):
        NKIPyKernel(hinted, "hlo").specialize(x)                             # default backend warns
    gk = NKIPyKernel(hinted, "nkigen").specialize(x)
    assert any(n.attrs.get("_knob", {}).get("mem_space") == "Shared" for n in gk.nodes)


def test_custom_op_reference_alias_and_inline():
    from nkipy_b200.core.cuda_op import cuda_custom_op

    src = 'extern "C" __global__ void scale_add_kernel(const float* a, const float* b, float* out) { int i = blockIdx.x * blockDim.x + threadIdx.x; if (i < 32) out[i] = 2.f * a[i] + b[i]; }'
    op = cuda_custom_op("scale_add", src, "scale_add_kernel", [((32,), "f32")], grid=(1,), block=(32,),
                        reference=lambda a, b: 2 * a + b)
    a, b = f32(32), f32(32)

    def k(x, y):
        return op(x, y) + 1

    np.testing.assert_allclose(k(a, b), 2 * a + b + 1, rtol=1e-6)             # direct mode -> reference
    from nkipy_b200.core.trace import NKIPyKernel

    g = NKIPyKernel(k, "hlo").specialize(a, b)
    assert any(n.opcode == "custom_call" and n.attrs["entry"] == "scale_add_kernel" for n in g.nodes)
    np.testing.assert_allclose(evaluate(g, [a, b])[0], 2 * a + b + 1, rtol=1e-6)
    from nkipy_b200.compiler.codegen import lower_to_cuda

    assert "scale_add_kernel" in lower_to_cuda(g)
    inplace = cuda_custom_op("bump", src, "scale_add_kernel", [((32,), "f32")], reference=lambda a, b: 2 * a + b,
                             aliases={0: 0})

    def k2(x, y):
        inplace(x, y)

    g2 = NKIPyKernel(k2, "hlo").specialize(a.copy(), b)
    assert g2.aliases and g2.outputs[0].name == "x"
    with pytest.raises(ValueError):
        cuda_custom_op("bad", src, "e", [])
