"""Loops are one node whatever the trip count, every pass also runs on the body, and the code generator expands
the iterations only when it emits launches."""
import json

import numpy as np

from nkipy_b200 import nkigen
from nkipy_b200.compiler.codegen import generate
from nkipy_b200.core.interp import evaluate
from nkipy_b200.core.ir import Graph, expand_loops, loop_body
from nkipy_b200.nkigen import apply_complete_knob_pipeline, trace

from ..harness import run_kernel_test

R = np.random.default_rng(9)


def _scan(trips):
    @trace(input_specs=[((trips, 8), "f32"), ((8, 8), "f32")])
    def k(x, w):
        def body(i, carry):
            h, s = carry
            h = np.tanh(h @ w + x[i] * 1.0)
            return h, s + np.sum(h)

        h, s = nkigen.fori_loop(0, trips, body, (np.zeros(8, np.float32), np.zeros((), np.float32)))
        return h, s

    return k


def test_ir_size_does_not_depend_on_the_trip_count():
    n4 = len(_scan(4).graph().nodes)
    n64 = len(_scan(64).graph().nodes)
    assert n4 == n64 and any(n.opcode == "loop" for n in _scan(64).graph().nodes)
    assert len(_scan(64).to_ir()) < 1.1 * len(_scan(4).to_ir()) + 64


def test_loop_matches_direct_mode_before_and_after_every_pass():
    k = _scan(16)
    x, w = R.standard_normal((16, 8)).astype(np.float32), (R.standard_normal((8, 8)) * 0.3).astype(np.float32)
    g = run_kernel_test(k, [x, w], rtol=1e-4, atol=1e-5)
    loop = next(n for n in g.nodes if n.opcode == "loop")
    body_ops = [n.opcode for n in loop_body(loop).nodes]
    assert "mul" not in body_ops                                # x[i] * 1.0 was canonicalised inside the body
    assert any("_tile" in n.attrs for n in loop_body(loop).nodes)   # the layout passes annotated the body's dot


def test_codegen_expands_iterations():
    k = _scan(3)
    g = Graph.from_text(apply_complete_knob_pipeline(k.to_ir()))
    plan = json.loads(generate(g).plan_json())
    assert sum("gemm" in l["kernel"] for l in plan["launches"]) == 3
    x, w = R.standard_normal((3, 8)).astype(np.float32), R.standard_normal((8, 8)).astype(np.float32)
    for a, b in zip(evaluate(expand_loops(g), [x, w]), evaluate(g, [x, w])):
        np.testing.assert_allclose(a, b, rtol=1e-6)


def test_static_index_use_falls_back_to_unrolling_and_direct_mode_is_a_python_loop():
    @trace(input_specs=[((6, 4), "f32")])
    def k(x):
        def body(i, acc):
            return acc + np.sum(x[i:i + 2], axis=0)      # slice bounds need a Python integer

        return nkigen.fori_loop(0, 4, body, np.zeros(4, np.float32))

    x = R.standard_normal((6, 4)).astype(np.float32)
    g = k.graph()
    assert not any(n.opcode == "loop" for n in g.nodes)
    np.testing.assert_allclose(evaluate(g, [x])[0], k(x), rtol=1e-6)
