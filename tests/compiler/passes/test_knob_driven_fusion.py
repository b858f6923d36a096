"""knob-driven-fusion groups same-shape elementwise ops and marks the direct consumer of a dot as its epilogue;
the code generator then compiles that chain into the GEMM kernel: matmul + bias + SiLU is ONE launch."""
import json

import numpy as np

from nkipy_b200.compiler.codegen import generate
from nkipy_b200.core.ir import Graph
from nkipy_b200.nkigen import apply_complete_knob_pipeline, trace

from ..harness import node, run_kernel_test

R = np.random.default_rng(7)


@trace(input_specs=[((256, 512), "bf16"), ((384, 512), "bf16"), ((384,), "bf16")])
def mlp(x, w, b):
    z = x @ w.T + b
    return z / (1.0 + np.exp(-z))


def _inputs():
    import ml_dtypes

    bf = ml_dtypes.bfloat16
    return [R.standard_normal((256, 512)).astype(bf), (R.standard_normal((384, 512)) * 0.05).astype(bf),
            R.standard_normal(384).astype(bf)]


def test_groups_and_epilogue_marks():
    g = run_kernel_test(mlp, _inputs(), stop_after="knob-driven-fusion", rtol=3e-2, atol=3e-2)
    d = node(g, "dot")
    adds = [n for n in g.nodes if n.opcode == "add"]
    assert adds[0].attrs["_epilogue_of"] == d.attrs["_op_id"]
    groups = {n.attrs["_fuse_group"] for n in g.nodes if "_fuse_group" in n.attrs}
    assert len(groups) == 1                                   # bias add, negate, exp, add, divide: one group


def test_dot_bias_silu_is_one_launch_with_a_fused_epilogue():
    g = Graph.from_text(apply_complete_knob_pipeline(mlp.to_ir()))
    prog = generate(g)
    plan = json.loads(prog.plan_json())
    assert len(plan["launches"]) == 1
    ga = plan["launches"][0]["args"][2]["gemm_args"]
    assert ga["fused_epilogue"] == ["add", "neg", "exp", "add", "div"]
    # the epilogue's operands (bias, the constant one) follow the GEMM block as plain buffer arguments
    assert all("buffer" in a for a in plan["launches"][0]["args"][3:]) and len(plan["launches"][0]["args"]) >= 4
    assert "struct Epi_" in prog.source and "nkb::gemm_bf16_body<" in prog.source


def test_without_the_pipeline_nothing_is_fused():
    g = Graph.from_text(mlp.to_ir())
    plan = json.loads(generate(g).plan_json())
    assert len(plan["launches"]) >= 2                         # the GEMM, then separate pointwise kernels
    assert [a["gemm_args"]["fused_epilogue"] for l in plan["launches"] for a in l["args"] if "gemm_args" in a] == [[]]


def test_result_with_a_second_user_is_not_an_epilogue():
    @trace(input_specs=[((128, 64), "bf16"), ((96, 64), "bf16")])
    def k(x, w):
        y = x @ w.T
        return np.tanh(y), y

    g = Graph.from_text(apply_complete_knob_pipeline(k.to_ir()))
    plan = json.loads(generate(g).plan_json())
    ga = [a["gemm_args"] for l in plan["launches"] for a in l["args"] if "gemm_args" in a][0]
    assert ga["fused_epilogue"] == []
