"""prepare-arithmetic: x ** 2 becomes x * x; with fast-math a division by a constant becomes a multiplication
by its reciprocal (off by default: the result is not bit-identical)."""
import numpy as np

from nkipy_b200.nkigen import trace

from ..harness import run_kernel_test

R = np.random.default_rng(1)


def test_square_becomes_multiply():
    @trace(input_specs=[((8, 8), "f32")])
    def k(x):
        return x ** 2 + np.power(x, 3.0)

    run_kernel_test(k, [R.standard_normal((8, 8)).astype(np.float32)], passes=["prepare-arithmetic"], check="""
        CHECK: mul(
        CHECK-COUNT-1: pow(
    """, rtol=1e-5)


def test_constant_division_only_with_fast_math():
    @trace(input_specs=[((8, 8), "f32")])
    def k(x):
        return x / 4.0

    x = R.standard_normal((8, 8)).astype(np.float32)
    run_kernel_test(k, [x], passes=["prepare-arithmetic"], check="CHECK: div(\nCHECK-NOT: mul(")
    run_kernel_test(k, [x], passes=["prepare-arithmetic"], fast_math=True, check="CHECK: mul(\nCHECK-NOT: div(")


def test_division_by_tensor_is_kept():
    @trace(input_specs=[((8, 8), "f32"), ((8, 8), "f32")])
    def k(x, y):
        return x / y

    run_kernel_test(k, [R.standard_normal((8, 8)).astype(np.float32), (R.random((8, 8)) + 1).astype(np.float32)],
                    passes=["prepare-arithmetic"], fast_math=True, check="CHECK: div(")
