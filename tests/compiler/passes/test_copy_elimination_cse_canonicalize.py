"""eliminate-uninitialized-copies / eliminate-same-memspace-copy remove copies that protect nothing; cse merges
identical computations; canonicalize applies algebraic identities and removes dead code."""
import numpy as np

from nkipy_b200.nkigen import trace

from ..harness import run_kernel_test

R = np.random.default_rng(4)


def f32(*s):
    return R.standard_normal(s).astype(np.float32)


def test_copy_of_fresh_constant_is_removed():
    @trace(input_specs=[((4, 4), "f32")])
    def k(x):
        return x + np.copy(np.ones((4, 4), np.float32))

    run_kernel_test(k, [f32(4, 4)], passes=["eliminate-uninitialized-copies"], check="CHECK-NOT: copy(\nCHECK: add(")


def test_copy_of_single_use_temporary_is_removed_but_parameter_copy_stays():
    @trace(input_specs=[((4, 4), "f32")])
    def k(x):
        return np.copy(np.exp(x)), np.copy(x)

    run_kernel_test(k, [f32(4, 4)], passes=["eliminate-same-memspace-copy"], check="CHECK-COUNT-1: copy(")


def test_cse_merges_repeated_subexpressions():
    @trace(input_specs=[((8,), "f32")])
    def k(x):
        return np.exp(x) * 2 + np.exp(x) * 2

    run_kernel_test(k, [f32(8)], passes=["cse"], check="CHECK-COUNT-1: exp(\nCHECK-COUNT-1: mul(")


def test_canonicalize_identities_and_dead_code():
    @trace(input_specs=[((8,), "f32")])
    def k(x):
        unused = np.sin(x)          # noqa: F841 - dead on purpose
        return (x * 1.0 - 0.0) / 1.0 + x.astype(np.float32)

    run_kernel_test(k, [f32(8)], passes=["canonicalize"], check="""
        CHECK-NOT: sin(
        CHECK-NOT: mul(
        CHECK-NOT: div(
        CHECK: add(
    """)
