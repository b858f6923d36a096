"""canonicalize-reshape merges reshape chains and drops identity reshapes; simplify-linalg composes transposes
and drops identity permutations."""
import numpy as np

from nkipy_b200.nkigen import trace

from ..harness import run_kernel_test

R = np.random.default_rng(3)


def test_reshape_chain_collapses():
    @trace(input_specs=[((4, 6), "f32")])
    def k(x):
        return np.exp(x.reshape(2, 12).reshape(24).reshape(4, 6))

    run_kernel_test(k, [R.standard_normal((4, 6)).astype(np.float32)], passes=["canonicalize-reshape"], check="""
        CHECK-NOT: reshape(
        CHECK: exp(
    """)


def test_double_transpose_is_identity():
    @trace(input_specs=[((3, 5, 7), "f32")])
    def k(x):
        return np.transpose(np.transpose(x, (2, 0, 1)), (1, 2, 0)) + 1

    run_kernel_test(k, [R.standard_normal((3, 5, 7)).astype(np.float32)], passes=["simplify-linalg"],
                    check="CHECK-NOT: transpose(\nCHECK: add(")


def test_transposes_compose_into_one():
    @trace(input_specs=[((3, 5, 7), "f32")])
    def k(x):
        return np.transpose(np.transpose(x, (2, 0, 1)), (0, 2, 1)) * 2

    run_kernel_test(k, [R.standard_normal((3, 5, 7)).astype(np.float32)], passes=["simplify-linalg", "canonicalize"],
                    check="CHECK-COUNT-1: transpose(")
