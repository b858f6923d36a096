"""Indexing, slicing, slice assignment, aliasing and type promotion of the tracing frontend."""
import numpy as np
import pytest

from nkipy_b200.core import dtypes as D
from nkipy_b200.core.trace import NKIPyKernel
from utils import check, run_traced, trace_kernel

R = np.random.default_rng(1)


def f32(*shape):
    return R.standard_normal(shape).astype(np.float32)


X = f32(6, 8, 10)


@pytest.mark.parametrize("key", [
    np.s_[2], np.s_[-1], np.s_[1:4], np.s_[:, 2:7:2], np.s_[::2, ::3, ::4], np.s_[..., 3], np.s_[1, ..., 2:5],
    np.s_[..., :], np.s_[:, -3:], np.s_[::-1], np.s_[:, 6:1:-2], np.s_[None], np.s_[:, None, :, None],
    np.s_[None, 2, None], np.s_[..., None], np.s_[1:2, None, ..., 4], np.s_[np.int32(2)], np.s_[np.int64(-2), 1:3],
    np.s_[2:2], np.s_[5:100],
], ids=str)
def test_basic_indexing(key):
    check(lambda a: a[key] * 1.0, X)


@pytest.mark.parametrize("key", [
    np.s_[[0, 2, 5]], np.s_[:, [1, 1, 3]], np.s_[np.array([[0, 1], [4, 5]])], np.s_[:, :, np.array([9, 0])],
    np.s_[1, [2, 3]], np.s_[[0, 1], [2, 3]], np.s_[[0, 1], :, [2, 3]], np.s_[:, [0, 1], [2, 3]],
    np.s_[np.arange(6), np.arange(6)], np.s_[[0, -1], 2:4], np.s_[2:5, [0, 3], ::2], np.s_[0, :, [1, 2]],
    np.s_[..., [1, 2]], np.s_[[1, 2], ...], np.s_[:, None, [1, 2]],
], ids=str)
def test_advanced_indexing_layout_matches_numpy(key):
    check(lambda a: a[key] * 1.0, X)


def test_dynamic_index_tensors():
    idx = np.array([4, 0, 3], dtype=np.int32)
    check(lambda a, i: a[i], X, idx)
    check(lambda a, i: a[:, i], X, idx)
    check(lambda a, i: a[1:3, i, ::2], X, idx)
    check(lambda a, i: a[2, i], X, idx)
    check(lambda a, i: a[..., i], X, idx)
    check(lambda a, i: a[i[0]], X, idx)
    pos = np.array([2], dtype=np.int32)
    check(lambda a, i: a[np.arange(6), i] * 2, X[:, :, 0], np.array([1, 0, 7, 3, 2, 5], dtype=np.int32))
    check(lambda a, p: a[:, p], X, pos)
    # index derived from the tensor itself ("view as index")
    check(lambda a: a[np.argmax(a[:, 0, 0])], X)


def test_indexing_errors():
    with pytest.raises(IndexError):
        trace_kernel(lambda a: a[7], X)
    with pytest.raises(IndexError):
        trace_kernel(lambda a: a[0, 0, 0, 0], X)
    with pytest.raises(IndexError):
        trace_kernel(lambda a: a[..., 1, ...], X)
    with pytest.raises(NotImplementedError):
        trace_kernel(lambda a: a[a > 0], X)
    with pytest.raises(IndexError):
        trace_kernel(lambda a: a[[1.5]], X)
    with pytest.raises(IndexError):
        trace_kernel(lambda a: a[[9]], X)


def _assign(key, value_fn):
    def k(a, v):
        a[key] = value_fn(v)
        return a

    return k


@pytest.mark.parametrize("key,vshape", [
    (np.s_[0], (8, 10)), (np.s_[1:3], (2, 8, 10)), (np.s_[:, 2], (6, 10)), (np.s_[..., 0], (6, 8)),
    (np.s_[2, 3, 4], ()), (np.s_[::2], (3, 8, 10)), (np.s_[:, 1::3, ::5], (6, 3, 2)), (np.s_[-1, :, 2:4], (8, 2)),
    (np.s_[1:3], (1, 10)), (np.s_[:, :, 3], (1,)),
], ids=str)
def test_slice_assignment(key, vshape):
    v = f32(*vshape) if vshape else np.float32(3.5)
    if vshape:
        check(_assign(key, lambda t: t), X.copy(), v)
    else:
        def k(a):
            a[key] = 3.5
            return a
        check(k, X.copy())


def test_scalar_fill_and_tensor_index_assignment():
    def fill(a):
        a[1:4, :, ::2] = 0.0
        a[0] = 7
        return a

    check(fill, X.copy())
    idx = np.array([5, 1], dtype=np.int32)

    def scatter(a, i, v):
        a[:, i] = v
        return a

    check(scatter, X.copy(), idx, f32(6, 2, 10))

    def scatter_const(a, v):
        a[[0, 3]] = v
        return a

    check(scatter_const, X.copy(), f32(2, 8, 10))

    def dyn_row(a, p, v):
        a[p[0]] = v
        return a

    check(dyn_row, X.copy(), np.array([4], dtype=np.int32), f32(8, 10))

    def kv_write(cache, pos, k):
        cache[:, pos] = k
        return cache

    check(kv_write, f32(2, 16, 4), np.array([3], dtype=np.int32), f32(2, 1, 4))


# ------------------------------------------------------------------ aliasing
def test_alias_single_multi_noreturn_mixed():
    A, B, C = f32(16, 32), f32(16, 32), f32(16, 32)

    def single(a, b):
        a[0, :] = b[1, :]
        return a

    g = check(single, A.copy(), B)
    assert [(a.output_index, a.param_index, a.is_user_returned) for a in g.aliases] == [(0, 0, True)]
    assert g.inputs[0].name == "a.must_alias_input" and g.outputs[0].name == "a" and g.inputs[1].name == "b"

    def multi(a, b, c):
        a[0:1, :] = b[0:1, :]
        c[2:3, :] = b[2:3, :]
        return a, c

    g = check(multi, A.copy(), B, C.copy())
    assert [(a.output_index, a.param_index) for a in g.aliases] == [(0, 0), (1, 2)]
    assert [o.name for o in g.outputs] == ["a", "c"]

    def no_return(a, b):
        a[0, :] = b[1, :]

    g = trace_kernel(no_return, A.copy(), B)
    assert len(g.outputs) == 1 and g.auto_aliased_indices == {0} and g.outputs[0].name == "a"

    def mixed(a, b):
        a[0, :] = b[1, :]
        return a + b

    g, outs = run_traced(mixed, A.copy(), B)
    assert [o.name for o in g.outputs] == ["output0", "a"] and g.auto_aliased_indices == {1}
    expect_a = A.copy()
    expect_a[0] = B[1]
    np.testing.assert_allclose(outs[0], expect_a + B, atol=1e-6)
    np.testing.assert_allclose(outs[1], expect_a, atol=1e-6)

    def rebinding_is_not_mutation(a, b):
        a += b
        return a

    g = trace_kernel(rebinding_is_not_mutation, A, B)
    assert not g.aliases and g.outputs[0].name == "output0"


def test_kernel_wrapper_api():
    def k(a, scale=2.0, *, flag=True):
        return a * scale if flag else a

    kern = NKIPyKernel.trace(k)
    assert kern.__name__ == "k" and "k" in repr(kern)
    g1 = kern.specialize(f32(4), scale=3.0)
    g2 = kern.specialize(f32(4), scale=4.0)
    assert g1.content_hash("") != g2.content_hash("")            # comptime constants are part of the trace
    assert g1.content_hash("") == NKIPyKernel(k).specialize(f32(4), scale=3.0).content_hash("")
    assert g1.content_hash("-O1") != g1.content_hash("-O3")
    assert kern.specialize(f32(5), scale=3.0).content_hash("") != g1.content_hash("")
    assert kern.specialize(f32(4).astype(np.float16), scale=3.0).content_hash("") != g1.content_hash("")
    np.testing.assert_allclose(kern(np.ones(3, np.float32)), 2 * np.ones(3))       # direct mode
    with pytest.warns(UserWarning):
        assert NKIPyKernel(k, "cpu").specialize(f32(4)) is None
    with pytest.raises(ValueError):
        NKIPyKernel(k, "tpu")


# ------------------------------------------------------------------ type promotion
ALL = [np.bool_, np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32, np.uint64, np.float16,
       D.bfloat16, np.float32]


def test_promotion_lattice_is_symmetric_and_concrete():
    for a in ALL:
        for b in ALL:
            ab, ba = D.promote_types(np.dtype(a), np.dtype(b)), D.promote_types(np.dtype(b), np.dtype(a))
            assert ab == ba, (a, b)
            assert isinstance(ab, np.dtype)
        assert D.promote_types(np.dtype(a), np.dtype(a)) == np.dtype(a)


def test_weak_scalars_defer_to_tensors():
    f16 = np.zeros(2, np.float16)
    assert D.find_common_type(f16, 1.0) == np.float16 and D.find_common_type(2, f16) == np.float16
    assert D.find_common_type(np.zeros(2, np.int8), 3) == np.int8
    assert D.find_common_type(np.zeros(2, np.int32), 1.5) == np.float32
    assert D.find_common_type(np.zeros(2, np.bool_), 1) == np.int32
    assert D.find_common_type(np.zeros(2, np.bool_), 1.0) == np.float32
    assert D.find_common_type(np.zeros(2, D.bfloat16), 1.0) == D.bfloat16
    assert D.find_common_type(1, 2.0) == np.float32
    assert D.scalar_dtype(3) == np.int32 and D.scalar_dtype(3.0, np.float16) == np.float16


def test_strong_promotions_and_fp8_rules():
    P = lambda a, b: D.promote_types(np.dtype(a), np.dtype(b))
    assert P(np.float16, D.bfloat16) == np.float32
    assert P(np.int32, np.float16) == np.float16 and P(np.int64, D.bfloat16) == D.bfloat16
    assert P(np.uint8, np.int8) == np.int16 and P(np.uint32, np.int32) == np.int64
    assert P(np.uint64, np.int8) == np.float32
    assert P(D.float8_e5m2, np.float16) == np.float16 and P(D.float8_e4m3, np.float32) == np.float32
    with pytest.raises(TypeError):
        P(D.float8_e5m2, D.float8_e4m3)
    g = trace_kernel(lambda a, b: a + b, np.zeros(3, np.float16), np.zeros(3, D.bfloat16.type))
    assert g.outputs[0].dtype == np.float32
    g = trace_kernel(lambda a: (a > 0) * 2.5, np.zeros(3, np.float32))      # bool x python float
    assert g.outputs[0].dtype == np.float32
    g = trace_kernel(lambda a: a * 2, np.zeros(3, np.int8))
    assert g.outputs[0].dtype == np.int8
    g = trace_kernel(lambda a: a / 2, np.zeros(3, np.int32))
    assert g.outputs[0].dtype == np.float32


def test_ml_dtypes_constants_roundtrip():
    w = np.arange(6, dtype=np.float32).reshape(2, 3).astype(D.bfloat16.type)
    check(lambda a: a.astype(np.float32) + w.astype(np.float32), np.ones((2, 3), np.float32))
    g, (out,) = run_traced(lambda a: (a + w).astype(np.float32), np.ones((2, 3), D.bfloat16.type))
    np.testing.assert_allclose(out, 1 + np.arange(6).reshape(2, 3))
