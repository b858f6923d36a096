"""remove-redundant-zero-fill: additions of an all-zero splat disappear (the accumulator of a tensor-core tile
starts from zero by itself), nothing else changes."""
import numpy as np

from nkipy_b200.nkigen import trace

from ..harness import run_kernel_test

R = np.random.default_rng(0)


def test_zero_fill_before_matmul_accumulation_is_dropped():
    @trace(input_specs=[((32, 16), "f32"), ((16, 8), "f32")])
    def k(a, b):
        acc = np.zeros((32, 8), np.float32)
        return acc + a @ b

    g = run_kernel_test(k, [R.standard_normal((32, 16)).astype(np.float32), R.standard_normal((16, 8)).astype(np.float32)],
                        passes=["remove-redundant-zero-fill"], check="""
        CHECK: dot(
        CHECK-NOT: add(
        CHECK: return
    """)
    assert [n.opcode for n in g.nodes] == ["dot"]


def test_zero_on_either_side_and_nonzero_kept():
    @trace(input_specs=[((4, 4), "f32")])
    def k(x):
        return (np.zeros_like(x) + x) + (x + np.ones_like(x))

    run_kernel_test(k, [R.standard_normal((4, 4)).astype(np.float32)], passes=["remove-redundant-zero-fill"], check="""
        CHECK-COUNT-2: add(
    """)
