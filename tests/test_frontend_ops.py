"""Tracing frontend: every op family, direct mode vs interpreted trace."""
import numpy as np
import pytest

from nkipy_b200.core import ops, tensor_apis
from utils import check, run_traced, trace_kernel

R = np.random.default_rng(0)


def f32(*shape, scale=1.0):
    return (R.standard_normal(shape) * scale).astype(np.float32)


def pos(*shape):
    return (R.random(shape) + 0.5).astype(np.float32)


def test_config1_softmax_and_mlp():
    x = np.random.default_rng(0).standard_normal((128, 512)).astype(np.float32)

    def softmax(x):
        e = np.exp(x - np.max(x, axis=-1, keepdims=True))
        return e / np.sum(e, axis=-1, keepdims=True)

    g, (out,) = run_traced(softmax, x)
    ex = np.exp(x - x.max(-1, keepdims=True))
    np.testing.assert_allclose(out, ex / ex.sum(-1, keepdims=True), atol=1e-5)

    rng = np.random.default_rng(0)
    xm = rng.standard_normal((64, 256)).astype(np.float32)
    w1 = (rng.standard_normal((256, 1024)) * 0.02).astype(np.float32)
    w2 = (rng.standard_normal((1024, 256)) * 0.02).astype(np.float32)

    def mlp(x, w1, w2):
        h = x @ w1
        h = 0.5 * h * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (h + 0.044715 * h ** 3)))
        return h @ w2

    g, (out,) = run_traced(mlp, xm, w1, w2)
    np.testing.assert_allclose(out, mlp(xm, w1, w2), atol=1e-5)


UNARY = [np.abs, np.exp, np.sqrt, np.square, np.negative, np.sin, np.cos, np.tan, np.arctan, np.tanh, np.ceil,
         np.floor, np.rint, np.trunc, np.sign, np.reciprocal, np.log, np.log1p, np.log2, np.expm1]


@pytest.mark.parametrize("fn", UNARY, ids=lambda f: f.__name__)
def test_unary(fn):
    x = pos(8, 16) if fn in (np.sqrt, np.log, np.log1p, np.log2, np.reciprocal) else f32(8, 16)
    check(lambda a: fn(a), x)


BINARY = [np.add, np.subtract, np.multiply, np.divide, np.maximum, np.minimum, np.power, np.logaddexp, np.remainder,
          np.floor_divide]


@pytest.mark.parametrize("fn", BINARY, ids=lambda f: f.__name__)
def test_binary_and_broadcast(fn):
    a, b = pos(4, 1, 8), pos(3, 8)
    check(lambda x, y: fn(x, y), a, b)
    check(lambda x: fn(x, 2.0), a)
    check(lambda x: fn(1.5, x), a)


def test_operators_and_inplace_are_functional():
    def k(a, b):
        c = a + b * 2 - a / 3
        c += b
        c *= 0.5
        c -= 1
        return -c % 3 + abs(b) ** 2 + (a // 2)

    g = check(k, pos(5, 6), pos(5, 6))
    assert not g.aliases


@pytest.mark.parametrize("fn", [np.equal, np.not_equal, np.greater, np.greater_equal, np.less, np.less_equal])
def test_comparisons(fn):
    a, b = f32(6, 7), f32(6, 7)
    b[0] = a[0]
    check(lambda x, y: fn(x, y), a, b)
    check(lambda x, y: fn(x, y), a.astype(np.float16), b.astype(np.float16))


def test_logical_and_bitwise():
    a = R.integers(0, 3, (5, 9)).astype(np.int32)
    b = R.integers(0, 3, (5, 9)).astype(np.int32)
    check(lambda x, y: np.logical_and(x, y), a, b)
    check(lambda x, y: np.logical_or(x, y), a, b)
    check(lambda x, y: np.logical_xor(x, y), a, b)
    check(lambda x: np.logical_not(x), a)
    check(lambda x, y: (x & y) | (x ^ y), a.astype(np.uint8), b.astype(np.uint8))
    check(lambda x: ~x, a.astype(np.int8))
    check(lambda x: np.bitwise_not(x), a.astype(np.uint8))


@pytest.mark.parametrize("shape_a,shape_b", [((4, 5), (5, 6)), ((5,), (5, 3)), ((2, 5), (5,)), ((5,), (5,)),
                                             ((3, 4, 5), (5, 2)), ((3, 1, 4, 5), (2, 5, 6)), ((2, 3, 4), (2, 4, 5))])
def test_matmul_shapes(shape_a, shape_b):
    check(lambda a, b: np.matmul(a, b), f32(*shape_a), f32(*shape_b))
    check(lambda a, b: a @ b, f32(*shape_a), f32(*shape_b))


def test_matmul_invalid_and_dot():
    with pytest.raises(ValueError):
        trace_kernel(lambda a, b: a @ b, f32(3, 4), f32(5, 6))
    check(lambda a, b: np.dot(a, b), f32(4, 5), f32(5, 3))
    check(lambda a, b: np.dot(a, b), f32(5), f32(5))
    check(lambda a, b: np.dot(a, b), f32(2, 3, 5), f32(5, 4))


@pytest.mark.parametrize("fn", [np.sum, np.max, np.min, np.mean, np.prod])
@pytest.mark.parametrize("axis,keepdims", [(None, False), (0, False), (-1, True), ((0, 2), False), ((1, 2), True)])
def test_reductions(fn, axis, keepdims):
    x = (pos(3, 4, 5) if fn is np.prod else f32(3, 4, 5))
    check(lambda a: fn(a, axis=axis, keepdims=keepdims), x, rtol=1e-3)


def test_reduction_variants():
    x = f32(4, 6)
    check(lambda a: np.var(a, axis=1), x)
    check(lambda a: np.std(a, axis=0, keepdims=True), x)
    check(lambda a: np.var(a), x)
    check(lambda a: np.any(a > 1.5, axis=1), x)
    check(lambda a: np.all(a > -5, axis=0), x)
    check(lambda a: np.count_nonzero(a > 0, axis=1), x)
    check(lambda a: a.mean(axis=1) + a.sum(axis=1) + a.max(axis=1) + a.min(axis=1) + a.std(axis=1) + a.var(axis=1), x)
    check(lambda a: np.cumsum(a, axis=0), x)
    check(lambda a: np.cumsum(a, axis=1), x)
    check(lambda a: np.cumsum(a), x)
    check(lambda a: np.sum(a), (R.random((4, 5)) > 0.5))


@pytest.mark.parametrize("fn", [np.argmax, np.argmin])
def test_argminmax(fn):
    x = R.integers(0, 4, (5, 7)).astype(np.float32)     # many ties: first occurrence must win
    check(lambda a: fn(a, axis=0), x)
    check(lambda a: fn(a, axis=1, keepdims=True), x)
    check(lambda a: fn(a), x)
    check(lambda a: a.argmax(axis=1) + a.argmin(axis=1), x)
    g = trace_kernel(lambda a: fn(a, axis=1), x)
    assert g.outputs[0].dtype == np.int32


def test_transforms():
    x = f32(2, 3, 4)
    check(lambda a: np.reshape(a, (6, -1)), x)
    check(lambda a: a.reshape(4, 6).T, x)
    check(lambda a: np.transpose(a, (2, 0, 1)), x)
    check(lambda a: a.transpose(1, -1, 0), x)
    check(lambda a: np.swapaxes(a, 0, 2), x)
    check(lambda a: a.swapaxes(1, 2), x)
    check(lambda a: np.expand_dims(a, 1), x)
    check(lambda a: np.expand_dims(a, (0, -1)), x)
    check(lambda a: np.squeeze(np.expand_dims(a, 0)), x)
    check(lambda a: a.reshape(2, 1, 3, 4).squeeze(1), x)
    check(lambda a: np.broadcast_to(a[:, :1, :], (2, 3, 4)), x)
    check(lambda a: np.copy(a) + a.copy(), x)
    check(lambda a: np.repeat(a, 3, axis=1), x)
    check(lambda a: np.repeat(a, 2, axis=-1), x)
    check(lambda a: np.repeat(a, np.int64(2)), x)
    check(lambda a: np.tile(a, (2, 1, 3)), x)
    check(lambda a: np.tile(a, 2), x)
    check(lambda a: np.flip(a, axis=1), x)
    check(lambda a: np.flip(a), x)
    check(lambda a: np.roll(a, 2, axis=2), x)
    check(lambda a: np.roll(a, (1, -1), axis=(0, 2)), x)
    check(lambda a: np.roll(a, 5), x)
    check(lambda a: a.ravel() * 2, x)
    check(lambda a: a.astype(np.float16).astype(np.float32), x)
    check(lambda a: a.clip(-0.5, 0.5) + np.clip(a, None, 0.2) + np.clip(a, -0.1, None), x)
    with pytest.raises(ValueError):
        trace_kernel(lambda a: np.transpose(a, (0, 1)), x)
    with pytest.raises(ValueError):
        trace_kernel(lambda a: np.squeeze(a, axis=0), x)
    with pytest.raises(ValueError):
        trace_kernel(lambda a: a.reshape(5, -1), x)
    with pytest.raises(TypeError):
        trace_kernel(lambda a: np.repeat(a, [1, 2, 3], axis=1), x)


def test_concat_split_stack_pad_diff():
    a, b = f32(2, 3), f32(4, 3)
    check(lambda x, y: np.concatenate([x, y], axis=0), a, b)
    check(lambda x: np.concatenate([x, np.ones((1, 3), dtype=np.float32)], axis=0), a)
    check(lambda x: np.concatenate([x]), a)
    check(lambda x, y: np.concatenate([x, y.astype(np.float16)[:2]], axis=-1), a, b)
    check(lambda y: np.split(y, 2, axis=0)[1], b)
    check(lambda y: np.split(y, [1, 3], axis=0)[1] * 2, b)
    check(lambda y: np.split(y, 3, axis=-1)[2], b)
    check(lambda x: np.stack([x, x * 2], axis=0), a)
    check(lambda x: np.stack([x, x * 2], axis=-1), a)
    check(lambda x: np.pad(x, 1), a)
    check(lambda x: np.pad(x, ((1, 2), (0, 3)), constant_values=1.5), a)
    check(lambda x: np.pad(x, ((2, 1), (1, 1)), mode="edge"), a)
    check(lambda y: np.diff(y, axis=0), b)
    check(lambda y: np.diff(y, n=2, axis=0), b)
    check(lambda y: np.diff(y, axis=1, prepend=0.0, append=1.0), b)
    check(lambda x, y: np.diff(y, axis=0, prepend=x), a, b)


def test_creation_and_like():
    x = f32(3, 4)
    check(lambda a: a + np.zeros_like(a) + np.ones_like(a) * 2 + np.full_like(a, 3.0) + np.zeros_like(np.empty_like(a)), x)
    check(lambda a: np.zeros_like(a, dtype=np.int32) + 1, x)
    check(lambda a: a + tensor_apis.zeros((3, 4), dtype=np.float32) + tensor_apis.full((3, 4), 2.5), x)
    check(lambda a: a * tensor_apis.constant(2.0) + tensor_apis.constant(np.arange(4, dtype=np.float32)), x)
    check(lambda a: np.tril(a) + np.triu(a, 1) - np.tril(a, -1) * np.triu(a, -2), x)
    check(lambda a: np.diag(a) * 2, x)
    check(lambda a: np.diag(a, 1), x)
    check(lambda a: np.diag(a, -1), x)
    check(lambda a: np.diag(a[0]), x)
    check(lambda a: np.diag(a[0], -2), x)
    check(lambda a: np.trace(a) + np.trace(a, offset=1), x)
    check(lambda a: np.outer(a[0], a[1]), x)
    check(lambda a: np.linalg.norm(a) + np.linalg.norm(a, axis=1, keepdims=True), x)
    with pytest.raises(ValueError):
        trace_kernel(lambda a: np.linalg.norm(a, ord=3), x)


def test_where_take_put():
    x, y = f32(4, 6), f32(4, 6)
    idx = np.array([3, 0, 5, -1], dtype=np.int32)
    check(lambda a, b: np.where(a > b, a, b), x, y)
    check(lambda a: np.where(a > 0, a, 0.0), x)
    check(lambda a: np.where(a > 0, 1, -1), x)
    check(lambda a: np.where(np.array([[True], [False], [True], [False]]), a, -a), x)
    check(lambda a: np.take(a, idx, axis=1), x)
    check(lambda a, i: np.take(a, i, axis=1), x, np.array([1, 2], dtype=np.int32))
    check(lambda a: np.take(a, 2, axis=0), x)
    check(lambda a: np.take(a, np.array([0, 7, 23])), x)
    ia = R.integers(0, 6, (4, 2)).astype(np.int32)
    check(lambda a, i: np.take_along_axis(a, i, axis=1), x, ia)
    check(lambda a: np.take_along_axis(a, np.argmax(a, axis=1, keepdims=True), axis=1), x)

    def put(a, i):
        np.put_along_axis(a, i, 9.0, axis=1)
        return a

    check(put, x.copy(), ia[:, :1])

    def put_t(a, i, v):
        np.put_along_axis(a, i, v, axis=1)
        return a * 2

    check(put_t, x.copy(), ia[:, :1], f32(4, 1))


def test_topk_conv_softmax_rmsnorm():
    x = f32(3, 10)
    check(lambda a: tensor_apis.topk(a, 3)[0], x)
    check(lambda a: tensor_apis.topk(a, 3)[1], x)
    check(lambda a: tensor_apis.topk(a, 2, is_ascend=True)[0], x)
    g = trace_kernel(lambda a: tensor_apis.topk(a, 3)[1], x)
    assert g.outputs[0].dtype == np.uint32
    with pytest.raises(NotImplementedError):
        trace_kernel(lambda a: tensor_apis.topk(a, 2, axis=0), x)
    check(lambda a: tensor_apis.softmax(a, axis=-1), x)
    check(lambda a, w: tensor_apis.rms_norm(a, w, 1e-5), x, pos(10))
    img, w, b = f32(2, 4, 9, 9), f32(6, 4, 3, 3), f32(6)
    check(lambda i, k: tensor_apis.conv2d(i, k), img, w, rtol=1e-3)
    check(lambda i, k, bb: tensor_apis.conv2d(i, k, bb, stride=2, padding=1), img, w, b, rtol=1e-3)
    check(lambda i, k: tensor_apis.conv2d(i, k, stride=(1, 2), padding=(0, 1), dilation=2), img, w, rtol=1e-3)
    check(lambda i, k: tensor_apis.conv2d(i, k, groups=2), img, f32(6, 2, 3, 3), rtol=1e-3)
    check(lambda i, k: tensor_apis.conv3d(i, k, padding=1), f32(1, 2, 5, 6, 7), f32(3, 2, 3, 3, 3), rtol=1e-3)


def test_composite_patterns():
    x, y = f32(6, 8), f32(6, 8)
    check(lambda a: np.clip(a / 6 + 0.5, 0, 1), x)                               # hard sigmoid
    check(lambda a: np.log1p(np.exp(-np.abs(a))) + np.maximum(a, 0), x)          # softplus
    check(lambda a: np.max(a, -1) + np.log(np.sum(np.exp(a - np.max(a, -1, keepdims=True)), -1)), x)
    check(lambda a, b: np.sum(a * b, -1) / (np.linalg.norm(a, axis=-1) * np.linalg.norm(b, axis=-1)), x, y)
    check(lambda a: (a - a.mean(-1, keepdims=True)) / (a.std(-1, keepdims=True) + 1e-5), x)
    check(lambda a, b: np.sum(a * np.abs(b), -1) / np.sum(np.abs(b), -1), x, y)
    check(lambda a: np.round(a, 2) + np.round(a), x)
    check(lambda a: np.isnan(a / a) | ~np.isfinite(np.log(np.abs(a) * 0)), x)

    def rope(q, cos, sin):
        h = q.shape[-1] // 2
        q0, q1 = q[..., :h], q[..., h:]
        return np.concatenate([q0 * cos - q1 * sin, q1 * cos + q0 * sin], axis=-1)

    check(rope, f32(2, 5, 8), f32(5, 4), f32(5, 4))


def test_tensor_protocol():
    from nkipy_b200.core.tensor import NKIPyTensorRef

    seen = {}

    def k(a):
        seen["len"], seen["T"], seen["size"], seen["strides"] = len(a), a.T.shape, a.size, a.strides
        seen["ndim"], seen["dtype"] = a.ndim, a.dtype
        with pytest.raises(TypeError):
            np.asarray(a)
        with pytest.raises(NotImplementedError):
            np.arctan2(a, a)
        with pytest.raises(NotImplementedError):
            np.fft.fft(a)
        assert isinstance(a, NKIPyTensorRef)
        return a

    g = trace_kernel(k, f32(3, 5))
    assert seen == {"len": 3, "T": (5, 3), "size": 15, "strides": (20, 4), "ndim": 2, "dtype": np.float32}
    assert g.nodes[-1].opcode == "copy" and g.outputs[0].name == "output0"     # pass-through gets a copy


def test_dtype_sanitize_and_bool_outputs():
    with pytest.warns(UserWarning):
        g = trace_kernel(lambda a: a * 2, np.arange(6, dtype=np.float64).reshape(2, 3))
    assert g.inputs[0].dtype == np.float32
    with pytest.warns(UserWarning):
        g = trace_kernel(lambda a: a + 1, np.arange(6, dtype=np.int64))
    assert g.outputs[0].dtype == np.int32
    g = trace_kernel(lambda a: a > 0, f32(4))
    assert g.outputs[0].dtype == np.uint8


def test_source_locations_recorded():
    g = trace_kernel(lambda a: np.exp(a) + 1, f32(4))
    assert all(n.loc and n.loc[0].endswith("test_frontend_ops.py") for n in g.nodes)
    assert "test_frontend_ops.py" in g.to_text()


def test_collectives_shapes_and_cpu_semantics():
    from nkipy_b200.distributed import collectives as cc

    x = f32(128, 256)
    grp = [[0, 1]]
    g = trace_kernel(lambda a: cc.all_gather(a, all_gather_dim=0, replica_groups=grp), x)
    assert g.outputs[0].shape == (256, 256)
    g = trace_kernel(lambda a: cc.reduce_scatter(a, reduce_scatter_dim=1, replica_groups=grp), x)
    assert g.outputs[0].shape == (128, 128)
    g = trace_kernel(lambda a: cc.all_to_all(a, split_dimension=1, concat_dimension=0, replica_groups=grp), x)
    assert g.outputs[0].shape == (256, 128)
    g = trace_kernel(lambda a: cc.all_reduce(a, replica_groups=grp, reduce_op=np.maximum), x)
    assert g.nodes[-1].attrs["op"] == "maximum"
    np.testing.assert_allclose(cc.all_reduce(x, replica_groups=grp), x * 2)
    assert cc.all_gather(x, 0, grp).shape == (256, 256)
    assert cc.all_to_all(x, 1, 0, grp).shape == (256, 128)
    check(lambda a: cc.all_reduce(a, replica_groups=grp) + cc.reduce_scatter(a, 0, grp)[:1], x)
