"""knob-driven-tiling turns tiles into launch decisions (CTA tile, k-block, ring depth, split-K, persistent grid)
and the code generator emits exactly those: two traces of one matmul with different knobs produce different
`block_n` / `stages` in the launch plan, with equal numerics (interpreter here, device in tests/test_runtime_gpu.py)."""
import json

import numpy as np

from nkipy_b200.compiler.codegen import generate
from nkipy_b200.core.interp import evaluate
from nkipy_b200.core.ir import Graph
from nkipy_b200.nkigen import apply_complete_knob_pipeline, knob, trace

from ..harness import node, run_kernel_test

R = np.random.default_rng(6)


def _mm(tile):
    @trace(input_specs=[((256, 512), "bf16"), ((384, 512), "bf16")])
    def k(x, w):
        y = x @ w.T
        if tile:
            knob(y).tile_op(tile_size=tile)
        return y

    return k


def _gemm_args(kernel):
    g = Graph.from_text(apply_complete_knob_pipeline(kernel.to_ir()))
    plan = json.loads(generate(g).plan_json())
    args = [a["gemm_args"] for l in plan["launches"] for a in l["args"] if "gemm_args" in a]
    assert len(args) == 1
    launch = next(l for l in plan["launches"] if any("gemm_args" in a for a in l["args"]))
    return g, args[0], launch


def test_tiling_record_of_a_default_matmul():
    g = Graph.from_text(apply_complete_knob_pipeline(_mm(None).to_ir(), stop_after="knob-driven-tiling"))
    t = node(g, "dot").attrs["_tiling"]
    assert t["cta_tile"] == [128, 256] and t["k_block"] == 64 and t["persistent"] is True
    assert t["split_k"] >= 1 and 1 <= t["grid"] <= 148 and t["stages"] >= 2


def test_different_knobs_emit_different_kernels_with_equal_numerics():
    import ml_dtypes

    x = R.standard_normal((256, 512)).astype(ml_dtypes.bfloat16)
    w = R.standard_normal((384, 512)).astype(ml_dtypes.bfloat16)
    seen, outs = {}, []
    for tile in (None, [128, 64], [128, 128]):
        g, ga, launch = _gemm_args(_mm(tile))
        seen[str(tile)] = (ga["block_n"], ga["stages"], launch["smem"], launch["grid"][0])
        outs.append(evaluate(g, [x, w])[0].astype(np.float32))
    assert seen["None"][0] == 256 and seen["[128, 64]"][0] == 64 and seen["[128, 128]"][0] == 128
    assert len({v[1] for v in seen.values()}) >= 2          # the ring depth follows the tile
    assert len({v[2] for v in seen.values()}) >= 2          # ... and so does the dynamic shared memory
    assert seen["[128, 64]"][3] >= seen["None"][3]          # narrower tiles -> more CTAs (up to the SM count)
    for o in outs[1:]:
        np.testing.assert_array_equal(o, outs[0])


def test_small_problem_gets_split_k():
    @trace(input_specs=[((64, 8192), "bf16"), ((128, 8192), "bf16")])
    def k(x, w):
        return x @ w.T

    g = Graph.from_text(apply_complete_knob_pipeline(k.to_ir(), stop_after="knob-driven-tiling"))
    assert node(g, "dot").attrs["_tiling"]["split_k"] > 1


def test_elementwise_ops_get_a_launch_shape():
    @trace(input_specs=[((1000,), "f32")])
    def k(x):
        return np.exp(x)

    g = run_kernel_test(k, [R.standard_normal(1000).astype(np.float32)], stop_after="knob-driven-tiling", rtol=1e-5)
    assert node(g, "exp").attrs["_tiling"] == {"block": 256, "grid": 4}
