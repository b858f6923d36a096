"""The promotion lattice of the tracing frontend (nkipy_b200/core/dtypes.py), checked exhaustively over all
pairs and against the sample entries of the reference's table (tests/unit/test_type_promotion.py there).
Two documented differences: two weak operands meet at a weak type that becomes int32 / float32 instead of
raising, and float64 participates (it is narrowed to float32 when a kernel is traced) instead of raising."""
import itertools

import ml_dtypes
import numpy as np
import pytest

from nkipy_b200.core import dtypes as D
from nkipy_b200.core.compile import trace
from nkipy_b200.core.interp import evaluate

W_I, W_F = D.WeakInt, D.WeakFloat
STRONG = [np.dtype(t) for t in (np.bool_, np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32,
                                np.uint64, np.float16, np.float32, ml_dtypes.bfloat16, ml_dtypes.float8_e4m3fn,
                                ml_dtypes.float8_e5m2)]
FP8 = {np.dtype(ml_dtypes.float8_e4m3fn), np.dtype(ml_dtypes.float8_e5m2)}


def join(a, b):
    return D.concrete(D.promote_types(a, b))


def test_join_is_symmetric_and_idempotent():
    for a, b in itertools.product(STRONG + [W_I, W_F], repeat=2):
        if a in FP8 and b in FP8 and a != b:
            continue
        assert join(a, b) == join(b, a), (a, b)
    for a in STRONG:
        assert join(a, a) == a


def test_every_pair_has_a_concrete_result():
    for a, b in itertools.product(STRONG, repeat=2):
        if a in FP8 and b in FP8 and a != b:
            with pytest.raises(TypeError, match="no implicit promotion"):
                D.promote_types(a, b)
            continue
        out = join(a, b)
        assert isinstance(out, np.dtype) and out in STRONG
    for a in STRONG:
        for w in (W_I, W_F):
            assert join(a, w) in STRONG


def test_join_is_an_upper_bound():
    """The result of a pair absorbs either operand: join(join(a, b), a) == join(a, b)."""
    for a, b in itertools.product(STRONG, repeat=2):
        if a in FP8 and b in FP8 and a != b:
            continue
        j = join(a, b)
        if j in FP8 and (a in FP8) != (b in FP8):
            continue
        assert join(j, a) == j and join(j, b) == j, (a, b, j)


@pytest.mark.parametrize("a,b,want", [
    (np.bool_, np.int32, np.int32), (np.bool_, np.float32, np.float32),
    (np.bool_, W_I, np.int32), (np.bool_, W_F, np.float32),
    (W_I, np.int8, np.int8), (W_I, np.float32, np.float32), (W_I, np.uint16, np.uint16),
    (W_F, np.int32, np.float32), (W_F, np.float16, np.float16), (W_F, ml_dtypes.bfloat16, ml_dtypes.bfloat16),
    (W_F, np.uint8, np.float32),
    (np.int8, np.int16, np.int16), (np.int32, np.int64, np.int64), (np.uint8, np.uint32, np.uint32),
    (np.int8, np.uint8, np.int16), (np.int16, np.uint16, np.int32), (np.int32, np.uint32, np.int64),
    (np.int32, np.uint64, np.float32), (np.int64, np.uint64, np.float32),
    (np.float16, np.float32, np.float32), (np.float16, ml_dtypes.bfloat16, np.float32),
    (ml_dtypes.bfloat16, np.float32, np.float32),
    (np.int32, np.float16, np.float16), (np.int64, ml_dtypes.bfloat16, ml_dtypes.bfloat16),
    (np.uint8, np.float32, np.float32),
    (ml_dtypes.float8_e5m2, np.float16, np.float16), (ml_dtypes.float8_e4m3fn, np.float32, np.float32),
])
def test_sample_entries(a, b, want):
    assert join(a, b) == np.dtype(want)


def test_operand_classification():
    assert D.weak_type_of(True) == np.dtype(np.bool_)            # a Python bool is a strong bool, not an int
    assert D.weak_type_of(3) is W_I and D.weak_type_of(-7) is W_I
    assert D.weak_type_of(2.5) is W_F
    assert D.weak_type_of(np.float16(1)) == np.dtype(np.float16)  # numpy scalars are strong
    assert D.weak_type_of(np.int8(1)) == np.dtype(np.int8)
    assert D.weak_type_of(np.zeros(3, np.uint16)) == np.dtype(np.uint16)

    class HasDtypeClass:
        dtype = np.float32                                       # a type object, not a dtype instance

    assert D.weak_type_of(HasDtypeClass()) == np.dtype(np.float32)
    with pytest.raises(TypeError):
        D.weak_type_of("text")


@pytest.mark.parametrize("tensor_dt,scalar,want", [
    (np.bool_, 1, np.int32), (np.bool_, 1.0, np.float32), (np.float32, 2, np.float32), (np.float32, 2.0, np.float32),
    (np.int8, 2, np.int8), (np.int8, 2.0, np.float32), (np.float16, 3, np.float16), (ml_dtypes.bfloat16, 0.5,
                                                                                      ml_dtypes.bfloat16),
    (np.uint8, True, np.uint8),
])
def test_find_common_type_tensor_with_python_scalar(tensor_dt, scalar, want):
    t = np.zeros(4, dtype=tensor_dt)
    assert D.find_common_type(t, scalar) == np.dtype(want)
    assert D.find_common_type(scalar, t) == np.dtype(want)
    assert D.scalar_dtype(scalar, tensor_dt) == np.dtype(want)


def test_two_strong_operands():
    f32, i32 = np.zeros(2, np.float32), np.zeros(2, np.int32)
    assert D.find_common_type(f32, i32) == np.float32
    assert D.find_common_type(i32, i32) == np.int32
    assert D.find_common_type(np.zeros(2, np.float16), np.zeros(2, ml_dtypes.bfloat16)) == np.float32


def test_scalar_dtype_alone():
    assert D.scalar_dtype(True) == np.bool_ and D.scalar_dtype(42) == np.int32 and D.scalar_dtype(-2.5) == np.float32
    assert D.scalar_dtype(np.int16(5)) == np.int16 and D.scalar_dtype(np.float32(1)) == np.float32


def test_two_weak_operands_meet_weakly():
    assert D.promote_types(W_I, W_I) is W_I and D.promote_types(W_F, W_F) is W_F
    assert D.promote_types(W_I, W_F) is W_F
    assert D.find_common_type(1, 2) == np.int32 and D.find_common_type(1, 2.0) == np.float32


def test_sixty_four_bit_types_are_narrowed_at_trace_time():
    assert D.sanitize_dtype(np.float64) == np.float32 and D.sanitize_dtype(np.int64) == np.int32
    assert D.sanitize_dtype(np.uint64) == np.uint32 and D.sanitize_dtype(np.float16) == np.float16
    with pytest.warns(UserWarning):
        g = trace(lambda a: a * 2.0).specialize(np.ones(4, np.float64))
    assert g.outputs[0].dtype == np.float32 and "f64" not in g.to_text()


@pytest.mark.parametrize("dt,scalar", [(np.int8, 3), (np.float16, 2), (np.float16, 0.5), (np.int32, 1.5), (np.bool_, 2),
                                       (np.uint8, 1.0)])
def test_traced_result_dtype_matches_the_lattice(dt, scalar):
    x = (np.arange(6) % 2).astype(dt)
    g = trace(lambda a: a + scalar).specialize(x)
    (out,) = evaluate(g, [x])
    assert out.dtype == D.find_common_type(x, scalar)
    np.testing.assert_allclose(out.astype(np.float64), x.astype(np.float64) + scalar, rtol=1e-3)
