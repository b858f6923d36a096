"""Memory group: annotate-memory-space (values inside a fusion group stay in registers unless they escape),
legalize-layout (TMA / TMEM legality decides tcgen05 vs SIMT and records the TMA boxes), insert-spill-reload
(the shared-memory budget shrinks the ring, then the tile, then fails), one-shot-bufferize (buffer ids with
reuse and in-place updates), insert-memref-dealloc (last-use lists)."""
import json

import numpy as np
import pytest

from nkipy_b200.compiler.codegen import generate
from nkipy_b200.core.ir import Graph
from nkipy_b200.nkigen import apply_complete_knob_pipeline, trace

from ..harness import node, run_kernel_test

R = np.random.default_rng(8)


def f32(*s):
    return R.standard_normal(s).astype(np.float32)


def test_fused_intermediates_live_in_registers():
    @trace(input_specs=[((32, 32), "f32")])
    def k(x):
        a = np.exp(x)
        b = a * 2
        return b + 1, a

    g = run_kernel_test(k, [f32(32, 32)], stop_after="annotate-memory-space", rtol=1e-5)
    assert node(g, "exp").attrs["_mem"] == "Global"           # escapes: it is a result
    assert node(g, "mul").attrs["_mem"] == "Register"


def test_legalize_picks_the_tensor_core_path_only_when_tma_can_address_it():
    @trace(input_specs=[((256, 512), "bf16"), ((384, 512), "bf16")])
    def ok(x, w):
        return x @ w.T

    @trace(input_specs=[((64, 100), "f32"), ((100, 36), "f32")])
    def odd(a, b):
        return a @ b

    g = Graph.from_text(apply_complete_knob_pipeline(ok.to_ir(), stop_after="legalize-layout"))
    d = node(g, "dot")
    assert d.attrs["_path"] == "tcgen05" and d.attrs["_tma_box_a"] == [64, 128] and d.attrs["_swizzle"] == "128B"
    g2 = Graph.from_text(apply_complete_knob_pipeline(odd.to_ir(), stop_after="legalize-layout"))
    assert node(g2, "dot").attrs["_path"] == "simt"
    kinds = [l["kernel"] for l in json.loads(generate(Graph.from_text(apply_complete_knob_pipeline(odd.to_ir()))
                                                      ).plan_json())["launches"]]
    assert any("gemm_simt" in k for k in kinds)


def test_spill_pass_changes_the_emitted_ring_depth_and_shared_memory():
    @trace(input_specs=[((512, 1024), "bf16"), ((768, 1024), "bf16")])
    def mm(x, w):
        return x @ w.T

    def emitted(cap):
        g = Graph.from_text(apply_complete_knob_pipeline(mm.to_ir(), smem_capacity=cap))
        launch = json.loads(generate(g).plan_json())["launches"][0]
        return node(g, "dot").attrs, launch["args"][2]["gemm_args"], launch["smem"]

    full_attrs, full_args, full_smem = emitted(None)
    small_attrs, small_args, small_smem = emitted(70000)
    assert small_attrs["_stages"] < full_attrs["_stages"] and small_attrs["_smem_bytes"] <= 70000
    assert small_args["stages"] == small_attrs["_stages"] < full_args["stages"]
    assert small_smem < full_smem
    with pytest.raises(RuntimeError) as ei:
        apply_complete_knob_pipeline(mm.to_ir(), smem_capacity=20000)
    assert "insert-spill-reload" in str(ei.value)


def test_bufferize_reuses_and_updates_in_place_and_dealloc_lists_last_uses():
    @trace(input_specs=[((64, 64), "f32")])
    def k(x):
        a = np.sum(np.exp(x), axis=1, keepdims=True)
        b = x - a
        c = np.sum(np.exp(b), axis=1, keepdims=True)
        return b - c

    g = run_kernel_test(k, [f32(64, 64)], rtol=1e-4, atol=1e-4)
    bufs = [n.attrs["_buffer"] for n in g.nodes if "_buffer" in n.attrs]
    assert any(b >= 0 for b in bufs)
    produced = [n for n in g.nodes if n.attrs.get("_buffer", -1) >= 0 and n.opcode not in ("reshape", "broadcast")]
    assert len({n.attrs["_buffer"] for n in produced}) < len(produced)       # some buffer is used twice
    assert any("_last_use_of" in n.attrs for n in g.nodes)
