"""Behaviour catalogue of the tensor API: each case is a small NumPy function traced and interpreted, compared with
NumPy itself.  The list follows what the reference's tests/unit/test_tensor_api.py and
test_tensor_api_native_ops.py probe (composite patterns, shape utilities, reductions with dtype/keepdims variants,
padding, cumulative ops, triangular / diagonal helpers, tensor methods, operators, in-place updates)."""
import numpy as np
import pytest

from utils import check

pytestmark = pytest.mark.filterwarnings("ignore::RuntimeWarning")     # log of negatives / 1 / 0 are on purpose

R = np.random.default_rng(7)
A = R.standard_normal((4, 6)).astype(np.float32)
B = R.standard_normal((4, 6)).astype(np.float32)
P = (R.random((4, 6)) + 0.5).astype(np.float32)
V = R.standard_normal(6).astype(np.float32)
C3 = R.standard_normal((2, 3, 4)).astype(np.float32)
SQ = R.standard_normal((5, 5)).astype(np.float32)
I8 = R.integers(-100, 100, (4, 6)).astype(np.int8)
U8 = R.integers(0, 255, (4, 6)).astype(np.uint8)
I32 = R.integers(-50, 50, (4, 6)).astype(np.int32)

CASES = {
    # composite patterns
    "hard_sigmoid": (lambda x: np.clip(x / 6.0 + 0.5, 0.0, 1.0), [A]),
    "softplus": (lambda x: np.log1p(np.exp(-np.abs(x))) + np.maximum(x, 0.0), [A]),
    "log_sum_exp": (lambda x: np.log(np.sum(np.exp(x - np.max(x, -1, keepdims=True)), -1)) + np.max(x, -1), [A]),
    "cosine_similarity": (lambda a, b: np.sum(a * b, -1) / (np.linalg.norm(a, axis=-1) * np.linalg.norm(b, axis=-1)), [A, B]),
    "row_standardise": (lambda x: (x - np.mean(x, -1, keepdims=True)) / np.std(x, -1, keepdims=True), [A]),
    "coefficient_of_variation": (lambda x: np.std(x, axis=0) / np.mean(x, axis=0), [P]),
    "weighted_average": (lambda x, w: np.sum(x * w, -1) / np.sum(w), [A, np.abs(V) + 0.1]),
    "low_pass_filter": (lambda x: 0.25 * x[:, :-2] + 0.5 * x[:, 1:-1] + 0.25 * x[:, 2:], [A]),
    "diagonal_gather": (lambda x: x[np.arange(5), np.arange(5)], [SQ]),
    # shape utilities
    "expand_dims_int": (lambda x: np.expand_dims(x, 1), [A]),
    "expand_dims_list": (lambda x: np.expand_dims(x, (0, -1)), [A]),
    "squeeze_none": (lambda x: np.squeeze(x[:, :1]), [A]),
    "squeeze_method": (lambda x: x[:, :1].squeeze(1), [A]),
    "swapaxes": (lambda x: np.swapaxes(x, 0, 2), [C3]),
    "swapaxes_method": (lambda x: x.swapaxes(1, 2), [C3]),
    "stack": (lambda a, b: np.stack([a, b]), [A, B]),
    "stack_axis": (lambda a, b: np.stack([a, b], axis=-1), [A, B]),
    "concatenate_negative_axis": (lambda a, b: np.concatenate([a, b], axis=-1), [A, B]),
    "concatenate_single": (lambda a: np.concatenate([a], axis=0), [A]),
    "concatenate_numpy_constant": (lambda a: np.concatenate([a, np.ones((1, 6), np.float32)], axis=0), [A]),
    "split_equal": (lambda x: np.split(x, 3, axis=1)[1], [A]),
    "split_indices": (lambda x: np.split(x, [1, 4], axis=-1)[2], [A]),
    "reshape_minus_one": (lambda x: x.reshape(-1, 3), [A]),
    "ravel": (lambda x: x.ravel(), [A]),
    "transpose_negative": (lambda x: np.transpose(x, (-1, 0, 1)), [C3]),
    "repeat_negative_axis": (lambda x: np.repeat(x, 2, axis=-1), [A]),
    "tile": (lambda x: np.tile(x, (2, 1)), [A]),
    "flip": (lambda x: np.flip(x, axis=1), [A]),
    "roll_axis0": (lambda x: np.roll(x, 1, axis=0), [A]),
    "broadcast_to": (lambda v: np.broadcast_to(v, (3, 6)) * 2.0, [V]),
    "broadcast_to_same": (lambda x: np.broadcast_to(x, (4, 6)) + 1.0, [A]),
    "copy": (lambda x: np.copy(x) + 1.0, [A]),
    "copy_method": (lambda x: x.copy() * 2.0, [A]),
    # reductions
    "mean_none": (lambda x: np.mean(x), [A]),
    "max_keepdims": (lambda x: np.max(x, axis=0, keepdims=True), [A]),
    "min_axis": (lambda x: np.min(x, axis=1), [A]),
    "sum_axes": (lambda x: np.sum(x, axis=(0, 2)), [C3]),
    "prod": (lambda x: np.prod(x, axis=-1), [P]),
    "prod_method": (lambda x: x.prod(axis=0), [P]),
    "var": (lambda x: np.var(x, axis=-1, keepdims=True), [A]),
    "std_none": (lambda x: np.std(x), [A]),
    "mean_method": (lambda x: x.mean(-1), [A]),
    "any": (lambda x: np.any(x > 1.5, axis=-1), [A]),
    "count_nonzero": (lambda x: np.count_nonzero(x > 0, axis=-1), [A]),
    "argmax_axis0": (lambda x: np.argmax(x, axis=0), [A]),
    "argmin_none": (lambda x: np.argmin(x), [A]),
    "argmax_method": (lambda x: x.argmax(-1), [A]),
    "cumsum_axis0": (lambda x: np.cumsum(x, axis=0), [A]),
    "cumsum_middle": (lambda x: np.cumsum(x, axis=1), [C3]),
    "norm_default": (lambda x: np.linalg.norm(x), [A]),
    "norm_axis_keepdims": (lambda x: np.linalg.norm(x, axis=-1, keepdims=True), [A]),
    "trace": (lambda x: np.trace(x), [SQ]),
    # elementwise extras
    "clip_no_min": (lambda x: np.clip(x, None, 0.5), [A]),
    "clip_no_max": (lambda x: np.clip(x, -0.5, None), [A]),
    "clip_method": (lambda x: x.clip(-1.0, 1.0), [A]),
    "round": (lambda x: np.round(x), [A]),
    "round_decimals": (lambda x: np.round(x, 2), [A]),
    "isnan": (lambda x: np.isnan(np.log(x)), [A]),
    "isfinite": (lambda x: np.isfinite(1.0 / (x - x)), [A]),
    "mod_operator": (lambda a, b: a % (np.abs(b) + 0.5), [A, B]),
    "floor_divide_operator": (lambda a, b: a // (np.abs(b) + 0.5), [A, B]),
    "outer": (lambda a, b: np.outer(a, b), [V, V * 2]),
    "diff": (lambda x: np.diff(x, axis=-1), [A]),
    "diff_n2": (lambda x: np.diff(x, n=2, axis=-1), [A]),
    "where_scalar": (lambda x: np.where(x > 0, x, 0.0), [A]),
    "where_tensors": (lambda a, b: np.where(a > b, a, b), [A, B]),
    # padding and triangular helpers
    "pad_constant": (lambda x: np.pad(x, ((1, 2), (0, 1))), [A]),
    "pad_edge": (lambda x: np.pad(x, ((1, 1), (2, 0)), mode="edge"), [A]),
    "tril": (lambda x: np.tril(x), [SQ]),
    "triu_k": (lambda x: np.triu(x, 1), [SQ]),
    "tril_negative_k": (lambda x: np.tril(x, -1), [SQ]),
    "diag_1d": (lambda v: np.diag(v), [V]),
    "diag_2d": (lambda x: np.diag(x), [SQ]),
    "diag_negative_k": (lambda x: np.diag(x, -1), [SQ]),
    # gathers / scatters
    "take_numpy_index": (lambda x: np.take(x, np.array([2, 0, 3]), axis=0), [A]),
    "take_scalar": (lambda x: np.take(x, 1, axis=1), [A]),
    "take_along_axis": (lambda x, i: np.take_along_axis(x, i, axis=-1), [A, np.argsort(A, axis=-1).astype(np.int32)]),
    "sort_last_axis": (lambda x: np.sort(x, axis=-1), [A]),
    "sort_axis0": (lambda x: np.sort(x, axis=0), [A]),
    "sort_flattened": (lambda x: np.sort(x, axis=None), [A]),
    "argsort_middle_axis": (lambda x: np.argsort(x, axis=1), [C3]),
    "argsort_then_gather": (lambda x: np.take_along_axis(x, np.argsort(x, axis=-1), axis=-1), [A]),
    "take_along_axis_constant": (lambda x: np.take_along_axis(x, np.array([[0], [2], [5], [1]]), axis=-1), [A]),
    # integer and bitwise
    "bitwise_and_or_xor": (lambda a, b: (a & b) | (a ^ b), [I32, I32[::-1].copy()]),
    "invert_u8": (lambda a: ~a, [U8]),
    "abs_i8": (lambda a: np.abs(a // 2), [I8]),
    # operators, methods, promotion
    "operators": (lambda a, b: (-a + b * 2 - a / 3) ** 2, [A, B]),
    "comparisons": (lambda a, b: ((a < b) & (a != b)) | (a >= 1.0), [A, B]),
    "matmul_1d_promotion": (lambda a, v: a @ v, [A, V]),
    "dot_1d": (lambda a, b: np.dot(a, b), [V, V * 3]),
    "matmul_batched": (lambda a, b: a @ b, [C3, C3.transpose(0, 2, 1).copy()]),
    "astype": (lambda x: x.astype(np.int32).astype(np.float32) * 0.5, [A * 10]),
    "bool_times_scalar": (lambda x: (x > 0) * 2.5, [A]),
    "mixed_dtype_sum": (lambda a, b: np.sum(a, -1) + np.sum(b, -1), [A, I32]),
    "zeros_like_override": (lambda x: np.zeros_like(x, dtype=np.int32) + 3, [A]),
    "ones_like": (lambda x: np.ones_like(x) * x, [A]),
    "full_like": (lambda x: np.full_like(x, 2.5) - x, [A]),
    "T_property": (lambda x: x.T @ x, [A]),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_catalogue(name):
    fn, inputs = CASES[name]
    check(fn, *[a.copy() for a in inputs], rtol=2e-4, atol=2e-4)


def test_in_place_operators_match_numpy_and_slice_assignment_aliases_the_parameter():
    def inplace(x, y):
        x += y
        x *= 2.0
        x -= 1.0
        return x

    check(inplace, A.copy(), B.copy())

    def assign(x, y):
        x[:, :2] = y[:, :2] * 3.0           # writes through the parameter: it comes back as an aliased output
        return np.sum(x, axis=-1)

    g = check(assign, A.copy(), B.copy())
    assert [o.name for o in g.outputs] == ["output0", "x"] and g.aliases


def test_len_shape_and_strides_are_trace_time_numbers():
    def kernel(x):
        assert len(x) == 4 and x.shape == (4, 6) and x.ndim == 2 and x.size == 24
        return x * float(len(x))

    check(kernel, A.copy())


def test_invalid_requests_are_rejected_while_tracing():
    with pytest.raises(Exception):
        check(lambda x: np.transpose(x, (0, 5)), A.copy())
    with pytest.raises(Exception):
        check(lambda x: np.squeeze(x, axis=0), A.copy())            # axis 0 has extent 4
    with pytest.raises(Exception):
        check(lambda a, b: a @ b, A.copy(), B.copy())               # inner dimensions differ
