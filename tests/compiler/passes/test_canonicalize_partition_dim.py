"""canonicalize-partition-dim: a transposed matmul operand is folded into the dot's contracting dimension and
the operand majors (K or MN) are recorded, so the code generator can pick a shared-memory layout instead of
materialising the transpose."""
import numpy as np

from nkipy_b200.nkigen import trace

from ..harness import node, run_kernel_test

R = np.random.default_rng(2)


def f32(*s):
    return R.standard_normal(s).astype(np.float32)


def test_transposed_rhs_is_folded():
    @trace(input_specs=[((16, 32), "f32"), ((24, 32), "f32")])
    def k(a, w):
        return a @ w.T

    g = run_kernel_test(k, [f32(16, 32), f32(24, 32)], passes=["canonicalize-partition-dim"], check="""
        CHECK-NOT: transpose(
        CHECK: dot(
    """)
    d = node(g, "dot")
    assert d.attrs["rhs_contract"] == [1] and d.attrs["_b_major"] == "K" and d.attrs["_a_major"] == "K"


def test_plain_matmul_records_mn_major_rhs():
    @trace(input_specs=[((16, 32), "f32"), ((32, 24), "f32")])
    def k(a, b):
        return a @ b

    g = run_kernel_test(k, [f32(16, 32), f32(32, 24)], passes=["canonicalize-partition-dim"])
    assert node(g, "dot").attrs["_b_major"] == "MN"


def test_transpose_with_other_users_stays():
    @trace(input_specs=[((16, 32), "f32"), ((24, 32), "f32")])
    def k(a, w):
        wt = w.T
        return a @ wt, wt * 2

    run_kernel_test(k, [f32(16, 32), f32(24, 32)], passes=["canonicalize-partition-dim"], check="CHECK: transpose(")
