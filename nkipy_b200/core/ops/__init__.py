"""Frontend operations: one dispatching `Op` object per operation.

The set and the names match the reference registry
(nkipy/src/nkipy/core/ops/__init__.py:180-306).  Primitive ops have an IR lowering
(registered under backend "hlo", see `_ir_impls`); ops that can be written with
other ops have a backend-agnostic composed implementation; ops without a NumPy
equivalent (`topk`, `softmax`, `rms_norm`, `conv2d/3d`, creation helpers and the four
collectives) also have a CPU implementation so kernels using them run unchanged in
CPU direct mode.  `softmax` and `rms_norm` over the last axis trace to one node each (one row kernel on the
device); for other axes, and in direct mode, they are compositions of primitives.  `erf` / `rsqrt` / `all`
exist as extra primitives.
"""

from __future__ import annotations

import math

import numpy as np

from ..backend import get_backend, set_source_location
from ._registry import Op

_NAMES = [
    # binary
    "add", "subtract", "multiply", "divide", "power", "maximum", "minimum", "bitwise_and", "bitwise_or",
    "bitwise_xor", "equal", "not_equal", "greater", "greater_equal", "less", "less_equal", "logical_and",
    "logical_or", "logical_xor", "logaddexp", "remainder", "floor_divide",
    # unary
    "abs", "exp", "log", "sqrt", "square", "negative", "reciprocal", "sin", "cos", "tan", "arctan", "tanh", "ceil",
    "floor", "rint", "trunc", "sign", "invert", "bitwise_not", "logical_not", "clip", "log1p", "log2", "expm1",
    "round_", "isnan", "isfinite", "erf", "rsqrt", "sigmoid", "gelu", "silu",
    # creation
    "constant", "zeros", "ones", "full", "zeros_like", "ones_like", "empty_like", "full_like", "tril", "triu", "diag",
    # linalg
    "dot", "matmul", "norm", "outer", "trace",
    # reduction
    "sum", "max", "min", "mean", "any", "all", "var", "std", "argmax", "argmin", "cumsum", "prod", "count_nonzero",
    # transform
    "reshape", "transpose", "expand_dims", "concatenate", "split", "copy", "repeat", "broadcast_to", "copyto",
    "astype", "squeeze", "pad", "swapaxes", "stack", "diff", "flip", "tile", "roll",
    # nn
    "softmax", "topk", "rms_norm", "sort", "argsort",
    # conv
    "conv2d", "conv3d",
    # indexing
    "where", "take", "take_along_axis", "put_along_axis", "scatter_along_axis", "static_slice",
    "dynamic_update_slice", "scatter_strided",
    # collectives
    "all_gather", "all_reduce", "reduce_scatter", "all_to_all",
]

for _n in _NAMES:
    globals()[_n] = Op(_n.rstrip("_") if _n == "round_" else _n)

__all__ = ["Op", "get_backend", "set_source_location"] + _NAMES


# --------------------------------------------------------------------------- IR lowerings
def _register_ir():
    from . import _ir_impls as I

    table = {
        "add": I.add, "subtract": I.subtract, "multiply": I.multiply, "divide": I.divide, "power": I.power,
        "maximum": I.maximum, "minimum": I.minimum, "bitwise_and": I.bitwise_and, "bitwise_or": I.bitwise_or,
        "bitwise_xor": I.bitwise_xor, "equal": I.equal, "not_equal": I.not_equal, "greater": I.greater,
        "greater_equal": I.greater_equal, "less": I.less, "less_equal": I.less_equal, "logical_and": I.logical_and,
        "logical_or": I.logical_or, "logical_xor": I.logical_xor,
        "abs": I.abs_, "exp": I.exp, "log": I.log, "sqrt": I.sqrt, "negative": I.negative, "sin": I.sin,
        "cos": I.cos, "arctan": I.arctan, "tanh": I.tanh, "ceil": I.ceil, "floor": I.floor, "rint": I.rint,
        "sign": I.sign, "invert": I.invert, "bitwise_not": I.invert, "logical_not": I.logical_not,
        "isfinite": I.isfinite, "erf": I.erf, "rsqrt": I.rsqrt,
        "constant": I.constant, "zeros": I.zeros, "ones": I.ones, "full": I.full, "zeros_like": I.zeros_like,
        "ones_like": I.ones_like, "empty_like": I.empty_like, "full_like": I.full_like, "tril": I.tril,
        "triu": I.triu, "diag": I.diag,
        "dot": I.dot, "matmul": I.matmul,
        "sum": I.sum_, "max": I.max_, "min": I.min_, "any": I.any_, "all": I.all_, "argmax": I.argmax,
        "argmin": I.argmin, "prod": I.prod,
        "reshape": I.reshape, "transpose": I.transpose, "expand_dims": I.expand_dims, "concatenate": I.concatenate,
        "split": I.split, "copy": I.copy, "repeat": I.repeat, "broadcast_to": I.broadcast_to, "astype": I.astype,
        "squeeze": I.squeeze, "pad": I.pad, "swapaxes": I.swapaxes, "stack": I.stack, "flip": I.flip,
        "tile": I.tile, "roll": I.roll,
        "topk": I.topk, "conv2d": I.conv2d, "conv3d": I.conv3d, "softmax": I.softmax, "rms_norm": I.rms_norm,
        "where": I.where, "take": I.take, "take_along_axis": I.take_along_axis, "put_along_axis": I.put_along_axis,
        "scatter_along_axis": I.scatter_along_axis, "static_slice": I.static_slice,
        "dynamic_update_slice": I.dynamic_update_slice, "scatter_strided": I.scatter_strided,
        "all_gather": I.all_gather, "all_reduce": I.all_reduce, "reduce_scatter": I.reduce_scatter,
        "all_to_all": I.all_to_all,
    }
    for name, fn in table.items():
        globals()[name].impl("hlo")(fn)


_register_ir()


# --------------------------------------------------------------------------- CPU (direct mode)
def _cpu(name):
    return globals()[name].impl("cpu")


for _n, _f in {
    "add": np.add, "subtract": np.subtract, "multiply": np.multiply, "divide": np.divide, "power": np.power,
    "maximum": np.maximum, "minimum": np.minimum, "bitwise_and": np.bitwise_and, "bitwise_or": np.bitwise_or,
    "bitwise_xor": np.bitwise_xor, "equal": np.equal, "not_equal": np.not_equal, "greater": np.greater,
    "greater_equal": np.greater_equal, "less": np.less, "less_equal": np.less_equal, "logical_and": np.logical_and,
    "logical_or": np.logical_or, "logical_xor": np.logical_xor, "abs": np.abs, "exp": np.exp, "log": np.log,
    "sqrt": np.sqrt, "negative": np.negative, "sin": np.sin, "cos": np.cos, "arctan": np.arctan, "tanh": np.tanh,
    "ceil": np.ceil, "floor": np.floor, "rint": np.rint, "sign": np.sign, "invert": np.invert,
    "bitwise_not": np.invert, "logical_not": np.logical_not, "isfinite": np.isfinite, "dot": np.dot,
    "matmul": np.matmul, "sum": np.sum, "max": np.max, "min": np.min, "any": np.any, "all": np.all,
    "argmax": np.argmax, "argmin": np.argmin, "prod": np.prod, "reshape": np.reshape, "transpose": np.transpose,
    "expand_dims": np.expand_dims, "concatenate": np.concatenate, "split": np.split, "copy": np.copy,
    "repeat": np.repeat, "broadcast_to": np.broadcast_to, "squeeze": np.squeeze, "pad": np.pad,
    "swapaxes": np.swapaxes, "stack": np.stack, "flip": np.flip, "tile": np.tile, "roll": np.roll,
    "where": np.where, "take": np.take, "take_along_axis": np.take_along_axis, "tril": np.tril, "triu": np.triu,
    "diag": np.diag, "zeros_like": np.zeros_like, "ones_like": np.ones_like, "empty_like": np.zeros_like,
    "full_like": np.full_like,
}.items():
    globals()[_n].impl("cpu")(_f)


@_cpu("astype")
def _astype_cpu(x, dtype):
    return np.asarray(x).astype(dtype)


@_cpu("erf")
def _erf_cpu(x):
    return np.vectorize(math.erf, otypes=[np.asarray(x).dtype if np.asarray(x).dtype.kind == "f" else np.float32])(x)


@_cpu("rsqrt")
def _rsqrt_cpu(x):
    return 1.0 / np.sqrt(x)


@_cpu("constant")
def _constant_cpu(value, dtype=None):
    if isinstance(value, (int, np.integer)) and not isinstance(value, (bool, np.bool_)) and dtype is None:
        dtype = np.int32
    if isinstance(value, float) and dtype is None:
        dtype = np.float32
    return np.asarray(value, dtype=dtype)


@_cpu("zeros")
def _zeros_cpu(shape, dtype=np.float32):
    return np.zeros(shape, dtype=dtype)


@_cpu("ones")
def _ones_cpu(shape, dtype=np.float32):
    return np.ones(shape, dtype=dtype)


@_cpu("full")
def _full_cpu(shape, fill_value, dtype=None):
    if dtype is None:
        dtype = np.int32 if isinstance(fill_value, (int, np.integer)) and not isinstance(fill_value, bool) else (
            np.float32 if isinstance(fill_value, float) else None)
    return np.full(shape, fill_value, dtype=dtype)


@_cpu("put_along_axis")
def _put_along_axis_cpu(x, indices, values, axis):
    out = np.array(x, copy=True)
    np.put_along_axis(out, np.asarray(indices).astype(np.int64), values, axis)
    return out


@_cpu("scatter_along_axis")
def _scatter_along_axis_cpu(x, indices, values, axis):
    out = np.array(x, copy=True)
    sl = [slice(None)] * out.ndim
    sl[axis] = np.asarray(indices).astype(np.int64)
    out[tuple(sl)] = values
    return out


@_cpu("static_slice")
def _static_slice_cpu(x, start, limit, stride=None):
    stride = stride or [1] * len(start)
    return np.asarray(x)[tuple(slice(s, l, st) for s, l, st in zip(start, limit, stride))]


@_cpu("dynamic_update_slice")
def _dus_cpu(x, value, starts, strides=None, sizes=None, squeezed=None):
    out = np.array(x, copy=True)
    value = np.asarray(value)
    nd = out.ndim
    strides = list(strides) if strides is not None else [1] * nd
    sizes = list(sizes) if sizes is not None else list(value.shape)
    sl = tuple(slice(s, s + (n - 1) * st + 1 if n else s, st) for s, n, st in zip(starts, sizes, strides))
    target = out[sl].shape
    if value.shape != target:
        natural = [n for n, sq in zip(sizes, squeezed or [False] * nd) if not sq]
        value = np.broadcast_to(value, natural).reshape(target)
    out[sl] = value
    return out


globals()["scatter_strided"].impl("cpu")(lambda x, value, starts, strides, sizes: _dus_cpu(x, value, starts, strides,
                                                                                          sizes))


@_cpu("topk")
def _topk_cpu(x, k, axis=-1, is_ascend=False):
    x = np.asarray(x)
    if axis not in (-1, x.ndim - 1):
        raise NotImplementedError("topk is implemented for the last axis only")
    key = x.astype(np.float32)
    order = np.argsort(key if is_ascend else -key, axis=-1, kind="stable")[..., :k]
    return np.take_along_axis(x, order, axis=-1), order.astype(np.uint32)


def _conv_cpu(nsp):
    def run(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
        from ..interp import _conv

        tup = lambda v: [int(v)] * nsp if isinstance(v, (int, np.integer)) else [int(t) for t in v]
        x, weight = np.asarray(x), np.asarray(weight)
        if x.ndim != nsp + 2:
            raise ValueError(f"conv{nsp}d expects a {nsp + 2}-D input")
        return _conv(x, weight, None if bias is None else np.asarray(bias),
                     {"stride": tup(stride), "padding": tup(padding), "dilation": tup(dilation), "groups": groups},
                     np.result_type(x.dtype, weight.dtype))

    return run


globals()["conv2d"].impl("cpu")(_conv_cpu(2))
globals()["conv3d"].impl("cpu")(_conv_cpu(3))


# collectives in direct mode: one process, "every rank holds the same data"
@_cpu("all_gather")
def _all_gather_cpu(data, all_gather_dim, replica_groups, **kw):
    return np.concatenate([np.asarray(data)] * len(replica_groups[0]), axis=all_gather_dim)


@_cpu("all_reduce")
def _all_reduce_cpu(data, replica_groups, reduce_op=np.add, **kw):
    n = len(replica_groups[0])
    data = np.asarray(data)
    if reduce_op is np.add:
        return data * n
    if reduce_op is np.multiply:
        return data ** n
    return data.copy()


@_cpu("reduce_scatter")
def _reduce_scatter_cpu(data, reduce_scatter_dim, replica_groups, reduce_op=np.add, **kw):
    n = len(replica_groups[0])
    part = np.split(np.asarray(data), n, axis=reduce_scatter_dim)[0]
    if reduce_op is np.add:
        return part * n
    if reduce_op is np.multiply:
        return part ** n
    return part.copy()


@_cpu("all_to_all")
def _all_to_all_cpu(data, split_dimension, concat_dimension, replica_groups, **kw):
    n = len(replica_groups[0])
    parts = np.split(np.asarray(data), n, axis=split_dimension)
    return np.concatenate([parts[0]] * n, axis=concat_dimension)


# --------------------------------------------------------------------------- composed (any backend)
def _f(name):
    return globals()[name]


@logaddexp.composed_impl
def _logaddexp(x, y):
    m = maximum(x, y)
    return add(m, log(add(exp(subtract(x, m)), exp(subtract(y, m)))))


@floor_divide.composed_impl
def _floor_divide(x, y):
    return floor(divide(x, y))


@remainder.composed_impl
def _remainder(x, y):
    return subtract(x, multiply(floor(divide(x, y)), y))


@reciprocal.composed_impl
def _reciprocal(x):
    return divide(1.0, x)


@square.composed_impl
def _square(x):
    return multiply(x, x)


@tan.composed_impl
def _tan(x):
    return divide(sin(x), cos(x))


@trunc.composed_impl
def _trunc(x):
    return multiply(sign(x), floor(_f("abs")(x)))


@clip.composed_impl
def _clip(x, a_min=None, a_max=None, **kw):
    a_min = kw.get("min", a_min)
    a_max = kw.get("max", a_max)
    if a_min is None and a_max is None:
        raise ValueError("One of max or min must be given")
    if a_min is not None:
        x = maximum(x, a_min)
    if a_max is not None:
        x = minimum(x, a_max)
    return x


@log1p.composed_impl
def _log1p(x):
    return log(add(x, 1.0))


@log2.composed_impl
def _log2(x):
    return multiply(log(x), 1.0 / math.log(2.0))


@expm1.composed_impl
def _expm1(x):
    return subtract(exp(x), 1.0)


@round_.composed_impl
def _round(x, decimals=0):
    if decimals == 0:
        return rint(x)
    f = float(10 ** decimals)
    return divide(rint(multiply(x, f)), f)


@isnan.composed_impl
def _isnan(x):
    return not_equal(x, x)


@sigmoid.composed_impl
def _sigmoid(x):
    return divide(1.0, add(1.0, exp(negative(x))))


@silu.composed_impl
def _silu(x):
    return multiply(x, _sigmoid(x))


@gelu.composed_impl
def _gelu(x, approximate="tanh"):
    if approximate == "tanh":
        inner = multiply(math.sqrt(2.0 / math.pi), add(x, multiply(0.044715, multiply(multiply(x, x), x))))
        return multiply(multiply(0.5, x), add(1.0, tanh(inner)))
    return multiply(multiply(0.5, x), add(1.0, erf(multiply(x, 1.0 / math.sqrt(2.0)))))


def _count(x, axis):
    shape = x.shape
    if axis is None:
        return int(np.prod(shape, dtype=np.int64))
    axes = (axis,) if isinstance(axis, (int, np.integer)) else tuple(axis)
    n = 1
    for a in axes:
        n *= shape[a]
    return n


@mean.composed_impl
def _mean(x, axis=None, dtype=None, keepdims=False, **kw):
    n = _count(x, axis)
    s = _f("sum")(x, axis=axis, keepdims=keepdims)
    if s.dtype.kind in "iub":
        s = astype(s, np.float32)
    return divide(s, float(n))


@var.composed_impl
def _var(x, axis=None, dtype=None, ddof=0, keepdims=False, **kw):
    if x.dtype.kind in "iub":
        x = astype(x, np.float32)
    m = _mean(x, axis=axis, keepdims=True)
    d = subtract(x, m)
    n = _count(x, axis)
    return divide(_f("sum")(multiply(d, d), axis=axis, keepdims=keepdims), float(n - ddof))


@std.composed_impl
def _std(x, axis=None, dtype=None, ddof=0, keepdims=False, **kw):
    return sqrt(_var(x, axis=axis, ddof=ddof, keepdims=keepdims))


@count_nonzero.composed_impl
def _count_nonzero(x, axis=None, keepdims=False, **kw):
    return _f("sum")(astype(not_equal(x, 0), np.int32), axis=axis, keepdims=keepdims)


@cumsum.composed_impl
def _cumsum(x, axis=None, dtype=None, **kw):
    """Cumulative sum as a matmul with an upper-triangular matrix of ones along `axis`."""
    if axis is None:
        x = reshape(x, (-1,))
        axis = 0
    nd = len(x.shape)
    axis = axis % nd
    n = x.shape[axis]
    dt = x.dtype if x.dtype.kind == "f" else np.dtype(np.float32)
    tri = np.triu(np.ones((n, n), dtype=np.float32)).astype(dt)
    xm = swapaxes(x, axis, nd - 1) if axis != nd - 1 else x
    xm = astype(xm, dt) if xm.dtype != dt else xm
    out = matmul(xm, constant(tri) if get_backend() != "cpu" else tri)
    if axis != nd - 1:
        out = swapaxes(out, axis, nd - 1)
    if x.dtype.kind != "f":
        out = astype(out, x.dtype)
    return out


@norm.composed_impl
def _norm(x, ord=None, axis=None, keepdims=False):
    if ord is not None and ord not in (2, "fro"):
        raise ValueError(f"Invalid norm order {ord!r}: only the 2-norm / Frobenius norm is supported")
    if ord == "fro" and axis is not None and not isinstance(axis, (tuple, list)):
        raise ValueError("Invalid norm order 'fro' for vectors")
    return sqrt(_f("sum")(multiply(x, x), axis=axis, keepdims=keepdims))


@outer.composed_impl
def _outer(a, b):
    return multiply(reshape(a, (-1, 1)), reshape(b, (1, -1)))


@trace.composed_impl
def _trace(x, offset=0, axis1=0, axis2=1, dtype=None):
    nd = len(x.shape)
    a1, a2 = axis1 % nd, axis2 % nd
    if a1 == a2:
        raise ValueError("axis1 and axis2 cannot be the same")
    rest = [i for i in range(nd) if i not in (a1, a2)]
    xt = transpose(x, rest + [a1, a2])
    n, m = xt.shape[-2], xt.shape[-1]
    r = np.arange(n)[:, None]
    c = np.arange(m)[None, :]
    mask = (c == r + offset)
    sel = where(mask if get_backend() == "cpu" else constant(mask), xt, 0)
    out = _f("sum")(_f("sum")(sel, axis=-1), axis=-1)
    return astype(out, dtype) if dtype is not None else out


def _sorted_last_axis(x, axis, descending):
    nd = len(x.shape)
    if axis is None:
        x, axis, nd = reshape(x, (-1,)), 0, 1
    axis = axis % nd
    if axis != nd - 1:
        x = swapaxes(x, axis, nd - 1)
    vals, idx = topk(x, x.shape[-1], axis=-1, is_ascend=not descending)
    if axis != nd - 1:
        vals, idx = swapaxes(vals, axis, nd - 1), swapaxes(idx, axis, nd - 1)
    return vals, idx


@sort.composed_impl
def _sort(x, axis=-1, descending=False):
    """Sorted copy along `axis` (None = flattened): a full-length top-k, so it lowers to the same kernel."""
    return _sorted_last_axis(x, axis, descending)[0]


@argsort.composed_impl
def _argsort(x, axis=-1, descending=False):
    """Indices that sort `x` along `axis` (int32; ties keep their original order like NumPy's stable sort)."""
    return astype(_sorted_last_axis(x, axis, descending)[1], np.int32)


@diff.composed_impl
def _diff(x, n=1, axis=-1, prepend=None, append=None):
    nd = len(x.shape)
    axis = axis % nd
    parts = []
    for extra in (prepend,):
        if extra is not None:
            parts.append(_edge(extra, x, axis))
    parts.append(x)
    if append is not None:
        parts.append(_edge(append, x, axis))
    if len(parts) > 1:
        x = concatenate(parts, axis=axis)
    for _ in range(n):
        size = x.shape[axis]
        hi = take(x, np.arange(1, size, dtype=np.int32), axis=axis)
        lo = take(x, np.arange(0, size - 1, dtype=np.int32), axis=axis)
        x = subtract(hi, lo)
    return x


def _edge(v, x, axis):
    if not hasattr(v, "backend_tensor") and np.ndim(v) == 0:
        shape = list(x.shape)
        shape[axis] = 1
        return full(tuple(shape), v, x.dtype)
    return v


@softmax.composed_impl
def _softmax(x, axis=-1):
    m = _f("max")(x, axis=axis, keepdims=True)
    e = exp(subtract(x, m))
    return divide(e, _f("sum")(e, axis=axis, keepdims=True))


@rms_norm.composed_impl
def _rms_norm(x, weight=None, eps=1e-6, axis=-1):
    xf = astype(x, np.float32) if x.dtype != np.float32 else x
    ms = _mean(multiply(xf, xf), axis=axis, keepdims=True)
    y = multiply(xf, divide(1.0, sqrt(add(ms, eps))))
    if weight is not None:
        y = multiply(y, weight)
    return astype(y, x.dtype) if y.dtype != x.dtype else y


@copyto.composed_impl
def _copyto(dst, src, **kw):
    value = broadcast_to(astype(src, dst.dtype) if getattr(src, "dtype", None) != dst.dtype else src, dst.shape)
    if hasattr(dst, "_rebind"):
        dst._rebind(value)
        return None
    np.copyto(dst, value)
    return None
