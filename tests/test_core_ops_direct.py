"""Operation objects called directly on NumPy arrays (the CPU backend of the registry, what a kernel that calls
`ops.<name>` or `tensor_apis.<name>` runs in direct mode), against NumPy; and the same calls traced + interpreted.
Mirrors the reference's tests/unit/test_core_ops_direct.py."""
import numpy as np
import pytest

from nkipy_b200.core import ops, tensor_apis
from utils import check

R = np.random.default_rng(3)
A = R.standard_normal((4, 6)).astype(np.float32)
B = R.standard_normal((4, 6)).astype(np.float32)
P = (R.random((4, 6)) + 0.5).astype(np.float32)
I = R.integers(-9, 9, (4, 6)).astype(np.int32)
J = R.integers(1, 9, (4, 6)).astype(np.int32)

UNARY = ["abs", "exp", "log", "sqrt", "negative", "sin", "cos", "tan", "arctan", "tanh", "ceil", "floor", "rint", "trunc",
         "sign", "reciprocal", "square", "log1p", "log2", "expm1", "isnan", "isfinite"]
BINARY = ["add", "subtract", "multiply", "divide", "power", "maximum", "minimum", "logaddexp", "remainder",
          "floor_divide", "equal", "not_equal", "greater", "greater_equal", "less", "less_equal"]
INT_BINARY = ["bitwise_and", "bitwise_or", "bitwise_xor"]
LOGICAL = ["logical_and", "logical_or", "logical_xor"]


@pytest.mark.parametrize("name", UNARY)
def test_unary_ops(name):
    x = P if name in ("log", "sqrt", "reciprocal", "log1p", "log2") else A
    want = getattr(np, name)(x)
    np.testing.assert_allclose(getattr(ops, name)(x), want, rtol=1e-5, atol=1e-6)
    check(lambda a: getattr(ops, name)(a), x.copy())


@pytest.mark.parametrize("name", BINARY)
def test_binary_ops(name):
    a, b = (P, P[::-1].copy()) if name in ("power", "remainder", "floor_divide", "divide") else (A, B)
    np.testing.assert_allclose(getattr(ops, name)(a, b), getattr(np, name)(a, b), rtol=1e-5, atol=1e-6)
    check(lambda x, y: getattr(ops, name)(x, y), a.copy(), b.copy())


@pytest.mark.parametrize("name", INT_BINARY)
def test_integer_ops(name):
    assert np.array_equal(getattr(ops, name)(I, J), getattr(np, name)(I, J))
    check(lambda x, y: getattr(ops, name)(x, y), I.copy(), J.copy())
    assert np.array_equal(ops.invert(J), np.invert(J))


@pytest.mark.parametrize("name", LOGICAL)
def test_logical_ops(name):
    a, b = A > 0, B > 0
    assert np.array_equal(getattr(ops, name)(a, b), getattr(np, name)(a, b))
    assert np.array_equal(ops.logical_not(a), ~a)


def test_reductions():
    for name in ("sum", "max", "min", "mean", "prod", "var", "std"):
        for axis, keep in ((None, False), (0, False), (-1, True)):
            np.testing.assert_allclose(getattr(ops, name)(P, axis=axis, keepdims=keep),
                                       getattr(np, name)(P, axis=axis, keepdims=keep), rtol=1e-5)
    assert np.array_equal(ops.argmax(A, axis=-1), np.argmax(A, -1)) and np.array_equal(ops.argmin(A, axis=0), np.argmin(A, 0))
    assert np.array_equal(ops.any(A > 1, axis=-1), np.any(A > 1, -1)) and bool(ops.all(P > 0))
    np.testing.assert_allclose(ops.cumsum(A, axis=1), np.cumsum(A, 1), rtol=1e-5)
    assert np.array_equal(ops.count_nonzero(A > 0, axis=0), np.count_nonzero(A > 0, 0))


def test_linalg_and_nn():
    w = R.standard_normal((6, 3)).astype(np.float32)
    np.testing.assert_allclose(ops.matmul(A, w), A @ w, rtol=1e-5)
    np.testing.assert_allclose(ops.dot(A[0], B[0]), np.dot(A[0], B[0]), rtol=1e-5)
    np.testing.assert_allclose(ops.outer(A[0], B[0]), np.outer(A[0], B[0]), rtol=1e-6)
    np.testing.assert_allclose(ops.norm(A, axis=-1), np.linalg.norm(A, axis=-1), rtol=1e-5)
    np.testing.assert_allclose(ops.trace(A[:4, :4]), np.trace(A[:4, :4]), rtol=1e-5)
    e = np.exp(A - A.max(-1, keepdims=True))
    np.testing.assert_allclose(ops.softmax(A), e / e.sum(-1, keepdims=True), rtol=1e-5)
    np.testing.assert_allclose(tensor_apis.rms_norm(A, P[0], 1e-6), A / np.sqrt((A * A).mean(-1, keepdims=True) + 1e-6) * P[0],
                               rtol=1e-5)
    v, i = ops.topk(A, 2)
    np.testing.assert_allclose(v, -np.sort(-A, -1)[:, :2])
    v, i = ops.topk(A, 2, is_ascend=True)
    np.testing.assert_allclose(v, np.sort(A, -1)[:, :2])
    np.testing.assert_allclose(ops.sort(A, axis=0), np.sort(A, 0))
    assert np.array_equal(ops.argsort(A), np.argsort(A, -1, kind="stable"))
    for name, f in (("sigmoid", lambda x: 1 / (1 + np.exp(-x))), ("silu", lambda x: x / (1 + np.exp(-x))),
                    ("rsqrt", None)):
        x = P if name == "rsqrt" else A
        want = 1 / np.sqrt(x) if name == "rsqrt" else f(x)
        np.testing.assert_allclose(getattr(ops, name)(x), want, rtol=1e-5)


def test_transforms_creation_and_indexing():
    assert ops.reshape(A, (6, 4)).shape == (6, 4) and ops.transpose(A, (1, 0)).shape == (6, 4)
    assert ops.expand_dims(A, 0).shape == (1, 4, 6) and ops.squeeze(A[:1], 0).shape == (6,)
    assert ops.concatenate([A, B], axis=1).shape == (4, 12) and ops.stack([A, B]).shape == (2, 4, 6)
    assert [p.shape for p in ops.split(A, 3, axis=1)] == [(4, 2)] * 3
    assert ops.repeat(A, 2, axis=0).shape == (8, 6) and ops.tile(A, (1, 2)).shape == (4, 12)
    np.testing.assert_allclose(ops.flip(A, axis=0), A[::-1])
    np.testing.assert_allclose(ops.roll(A, 2, axis=1), np.roll(A, 2, 1))
    np.testing.assert_allclose(ops.pad(A, ((1, 0), (0, 2))), np.pad(A, ((1, 0), (0, 2))))
    np.testing.assert_allclose(ops.clip(A, -0.5, 0.5), np.clip(A, -0.5, 0.5))
    np.testing.assert_allclose(ops.where(A > 0, A, B), np.where(A > 0, A, B))
    np.testing.assert_allclose(ops.take(A, np.array([2, 0]), axis=0), A[[2, 0]])
    idx = np.argsort(A, -1)
    np.testing.assert_allclose(ops.take_along_axis(A, idx, axis=-1), np.take_along_axis(A, idx, -1))
    np.testing.assert_allclose(ops.tril(A[:4, :4]), np.tril(A[:4, :4]))
    np.testing.assert_allclose(ops.triu(A[:4, :4], 1), np.triu(A[:4, :4], 1))
    np.testing.assert_allclose(ops.diag(A[0]), np.diag(A[0]))
    assert ops.zeros((2, 3), np.float32).sum() == 0 and float(ops.full((2,), 4.0, np.float32)[0]) == 4.0
    assert ops.ones_like(A).dtype == np.float32 and ops.zeros_like(I).dtype == np.int32
    assert ops.astype(A, np.int32).dtype == np.int32 and ops.broadcast_to(A[0], (3, 6)).shape == (3, 6)
    np.testing.assert_allclose(ops.diff(A, axis=-1), np.diff(A, axis=-1), rtol=1e-6)
    np.testing.assert_allclose(ops.swapaxes(A, 0, 1), A.T)


def test_an_op_without_an_implementation_says_so():
    class Backendless:
        pass

    with pytest.raises(Exception):
        ops.add(Backendless(), 1)
