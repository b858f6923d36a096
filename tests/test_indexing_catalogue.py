"""Indexing and slicing catalogue: each case is traced and interpreted, compared with NumPy.  The list follows what
the reference's tests/unit/test_indexing_slicing_comprehensive.py probes: basic / stepped / nested slices, assignment,
array and list indices, static mixed with dynamic (traced) indices, negative indices, NumPy integer scalars, ellipsis
and newaxis in every position, and the error cases."""
import numpy as np
import pytest

from utils import check

R = np.random.default_rng(11)
X = R.standard_normal((6, 8)).astype(np.float32)
T3 = R.standard_normal((4, 5, 6)).astype(np.float32)
T4 = R.standard_normal((2, 3, 4, 5)).astype(np.float32)
IDX = np.array([3, 0, 5], np.int32)
IDX2 = np.array([1, 1, 4], np.int32)

CASES = {
    # basic, stepped and nested slices
    "row": (lambda x: x[2], [X]),
    "element": (lambda x: x[2, 3] * 2.0, [X]),
    "range": (lambda x: x[1:4], [X]),
    "two_ranges": (lambda x: x[1:4, 2:7], [X]),
    "step": (lambda x: x[::2, 1::3], [X]),
    "open_ended": (lambda x: x[:, 3:], [X]),
    "nested": (lambda x: x[1:5][1:3][:, 2:4], [X]),
    "negative_index": (lambda x: x[-1] + x[:, -2][:, None], [X]),
    "negative_slice": (lambda x: x[-4:-1, :-3], [X]),
    "numpy_int32_scalar": (lambda x: x[np.int32(2)], [X]),
    "numpy_int64_scalar": (lambda x: x[:, np.int64(5)], [X]),
    "slice_3d": (lambda t: t[1, :, 2:5], [T3]),
    "slice_then_index": (lambda t: t[:, 1:4][2, 0], [T3]),
    # ellipsis
    "ellipsis_identity": (lambda t: t[...] + 1.0, [T3]),
    "ellipsis_leading": (lambda t: t[..., 2], [T3]),
    "ellipsis_trailing": (lambda t: t[1, ...], [T3]),
    "ellipsis_middle": (lambda t: t[0, ..., 3], [T4]),
    "ellipsis_with_slice": (lambda t: t[..., 1:3, :], [T4]),
    # newaxis
    "newaxis_leading": (lambda x: x[None], [X]),
    "newaxis_trailing": (lambda x: x[:, :, None], [X]),
    "newaxis_multiple": (lambda x: x[None, :, None, :], [X]),
    "newaxis_with_int": (lambda x: x[2, None, :], [X]),
    "newaxis_with_ellipsis": (lambda t: t[..., None], [T3]),
    "newaxis_with_slice": (lambda x: x[1:3, None, ::2], [X]),
    # array and list indices
    "ndarray_index": (lambda x: x[np.array([4, 1, 1])], [X]),
    "list_index": (lambda x: x[[0, 5, 2]], [X]),
    "ndarray_index_axis1": (lambda x: x[:, np.array([7, 0])], [X]),
    "token_selection": (lambda t: t[:, np.array([0, 4]), :], [T3]),
    "head_selection": (lambda t: t[:, :, np.array([1, 3, 5])], [T3]),
    # dynamic (traced) indices
    "dynamic_rows": (lambda x, i: x[i], [X, IDX]),
    "dynamic_columns": (lambda x, i: x[:, i], [X, IDX]),
    "dynamic_with_static_slice": (lambda t, i: t[i, 1:4], [T3[:, :, :], np.array([3, 0], np.int32)]),
    "dynamic_with_static_int": (lambda t, i: t[2, i], [T3, np.array([4, 0, 1], np.int32)]),
    "dynamic_pair": (lambda x, i, j: x[i, j], [X, IDX, IDX2]),
    "view_as_index": (lambda x, i: x[i[1:]], [X, IDX]),
    "computed_index": (lambda x, i: x[(i + 1) % 6], [X, IDX]),
    # assignment
    "assign_scalar_slice": (lambda x: _assign(x, (slice(1, 3),), 0.5), [X]),
    "assign_row": (lambda x, v: _assign(x, (2,), v), [X, X[0] * 3]),
    "assign_block": (lambda x, v: _assign(x, (slice(0, 2), slice(4, 8)), v), [X, X[:2, :4] * -1]),
    "assign_step": (lambda x: _assign(x, (slice(None, None, 2),), 1.0), [X]),
    "assign_ellipsis": (lambda t: _assign(t, (Ellipsis, 0), 9.0), [T3]),
    "assign_negative": (lambda x, v: _assign(x, (-1,), v), [X, X[1] + 1]),
    "assign_dynamic_rows": (lambda x, i, v: _assign(x, (i,), v), [X, np.array([4, 1], np.int32), X[:2] * 2]),
    "assign_broadcast": (lambda x, v: _assign(x, (slice(None), slice(0, 3)), v), [X, X[:, :1] * 0 + 7]),
    "assign_then_read": (lambda x: _assign(x, (0,), 1.0)[0:2].sum(axis=0), [X]),
}


def _assign(x, key, value):
    y = x * 1.0                      # a fresh tensor, so that the caller's array is untouched in direct mode
    y[key if len(key) > 1 else key[0]] = value
    return y


@pytest.mark.parametrize("name", sorted(CASES))
def test_indexing(name):
    fn, inputs = CASES[name]
    check(fn, *[a.copy() for a in inputs])


def test_a_slice_of_a_traced_tensor_is_a_value_not_a_view():
    """Writing into a slice taken earlier does not reach the tensor it was taken from: slicing creates a new value in
    the graph (the reference's HLO mode behaves the same and skips its view-assignment test for that reason).  Writing
    through the tensor itself (`x[1:3] = ...`) is what updates it."""
    from utils import run_traced

    def through_slice(x):
        v = x[1:3]
        v[:] = 0.0
        return x.sum(), v.sum()

    _, out = run_traced(through_slice, X.copy())
    np.testing.assert_allclose(out[0], X.sum(), rtol=1e-5)
    assert float(out[1]) == 0.0

    def through_tensor(x):
        x[1:3] = 0.0
        return x.sum()

    g = check(through_tensor, X.copy())
    assert "x" in [o.name for o in g.outputs]                 # the parameter comes back as an aliased output


@pytest.mark.parametrize("bad", [lambda x: x[6], lambda x: x[:, 9], lambda x: x[0, 0, 0], lambda x: x[..., ...],
                                 lambda x: x[1.5]])
def test_error_cases(bad):
    with pytest.raises(Exception):
        check(bad, X.copy())
