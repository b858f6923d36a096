"""infer-layout: matmuls are seeded with the hardware tile (128 x up to 256 x 64, accumulator in tensor memory,
operands in shared memory), user knobs override the seed, elementwise consumers of a dot inherit its output
tile as epilogue candidates, other elementwise ops and reductions get a row tile in global memory."""
import numpy as np

from nkipy_b200.nkigen import knob, trace

from ..harness import node, run_kernel_test

R = np.random.default_rng(5)


def bf(*s):
    import ml_dtypes

    return R.standard_normal(s).astype(ml_dtypes.bfloat16)


def test_default_seed_and_propagation():
    @trace(input_specs=[((256, 512), "f32"), ((512, 384), "f32")])
    def k(a, b):
        return np.tanh(a @ b)

    g = run_kernel_test(k, [R.standard_normal((256, 512)).astype(np.float32),
                            R.standard_normal((512, 384)).astype(np.float32)], stop_after="infer-layout",
                        check='CHECK: "_tile": [128, 256, 64]', rtol=1e-4, atol=1e-4)
    d, t = node(g, "dot"), node(g, "tanh")
    assert d.attrs["_mem"] == "Tensor" and d.attrs["_operand_mem"] == "Shared"
    assert t.attrs["_tile"] == [128, 256] and t.attrs["_mem"] == "Register"


def test_small_n_picks_smaller_tile():
    @trace(input_specs=[((64, 128), "f32"), ((128, 48), "f32")])
    def k(a, b):
        return a @ b

    g = run_kernel_test(k, [R.standard_normal((64, 128)).astype(np.float32),
                            R.standard_normal((128, 48)).astype(np.float32)], stop_after="infer-layout", rtol=1e-4,
                        atol=1e-4)
    assert node(g, "dot").attrs["_tile"] == [64, 64, 64]


def test_knob_overrides_seed_and_mem_space_alias():
    @trace(input_specs=[((256, 512), "f32"), ((512, 384), "f32")])
    def k(a, b):
        c = a @ b
        knob(c).tile_op(tile_size=[128, 64], reduction_tile=[32])
        d = c * 2
        knob(d).layout(mem_space="Sbuf")
        return d

    g = run_kernel_test(k, [R.standard_normal((256, 512)).astype(np.float32),
                            R.standard_normal((512, 384)).astype(np.float32)], stop_after="infer-layout", rtol=1e-4,
                        atol=1e-4)
    assert node(g, "dot").attrs["_tile"] == [128, 64, 32]
    assert node(g, "mul").attrs["_mem"] == "Shared"


def test_reduction_tile_covers_reduced_axes():
    @trace(input_specs=[((16, 40), "f32")])
    def k(x):
        return np.sum(x, axis=1)

    g = run_kernel_test(k, [R.standard_normal((16, 40)).astype(np.float32)], stop_after="infer-layout", rtol=1e-5)
    assert node(g, "reduce").attrs["_tile"] == [1, 40]
