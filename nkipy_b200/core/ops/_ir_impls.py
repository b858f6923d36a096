"""IR lowerings of the primitive frontend operations (backend "hlo").

Each function takes traced tensors / NumPy arrays / Python scalars, appends nodes to
the graph of the active trace context and returns a new `NKIPyTensorRef`.  The
behaviours follow the reference's lowering layer
(nkipy/src/nkipy/core/ops/_hlo_impls.py): weak-type promotion then broadcast then
convert for binary ops, comparisons produce bool, logical ops compare against zero
first, reductions keep the input dtype, argmax/argmin return int32 with
first-occurrence semantics, matmul follows NumPy's 1-D promotion and batch
broadcasting, `take` wraps negative constant indices, `topk` works on the last axis
and returns uint32 indices, collectives change the shape along their dimension.
"""

from __future__ import annotations

import math
from typing import Any, List, Optional, Sequence, Tuple, Union

import numpy as np

from ..backend.hlo import get_hlo_context
from ..dtypes import (concrete, dtype_name, find_common_type, finfo_max, finfo_min, is_float, promote_types,
                      sanitize_dtype, weak_type_of)
from ..ir import Value
from ..tensor import NKIPyTensorRef

Tensor = NKIPyTensorRef


def G():
    return get_hlo_context().module


def wrap(v: Value) -> Tensor:
    return NKIPyTensorRef(v)


def is_tensor(x) -> bool:
    return isinstance(x, NKIPyTensorRef)


def const(arr) -> Value:
    arr = np.asarray(arr)
    arr = arr.astype(sanitize_dtype(arr.dtype), copy=False)
    return G().op("constant", value=np.require(arr, requirements="C"))


def convert(v: Value, dtype) -> Value:
    dtype = np.dtype(dtype)
    if v.dtype == dtype:
        return v
    return G().op("convert", v, dtype=dtype_name(dtype))


def as_value(x, dtype=None) -> Value:
    """IR value of any operand; Python scalars become 0-d constants of `dtype` (or their weak default)."""
    if is_tensor(x):
        v = x.backend_tensor
        return convert(v, dtype) if dtype is not None else v
    if isinstance(x, (bool, int, float, np.generic)) and not isinstance(x, np.ndarray):
        dt = np.dtype(dtype) if dtype is not None else concrete(weak_type_of(x))
        dt = sanitize_dtype(dt)
        return G().op("constant", value=np.asarray(x).astype(dt))
    arr = np.asarray(x)
    v = const(arr)
    return convert(v, dtype) if dtype is not None else v


def shape_of(x) -> Tuple[int, ...]:
    if is_tensor(x):
        return x.shape
    return tuple(np.shape(x))


def broadcast_value(v: Value, shape: Sequence[int]) -> Value:
    shape = tuple(int(s) for s in shape)
    if v.shape == shape:
        return v
    if len(v.shape) > len(shape):
        raise ValueError(f"cannot broadcast shape {v.shape} to {shape}")
    off = len(shape) - len(v.shape)
    for i, d in enumerate(v.shape):
        if d != 1 and d != shape[off + i]:
            raise ValueError(f"operands could not be broadcast together with shapes {v.shape} {shape}")
    return G().op("broadcast", v, shape=list(shape), dims=list(range(off, len(shape))))


def broadcast_pair(a: Value, b: Value) -> Tuple[Value, Value]:
    try:
        shape = np.broadcast_shapes(a.shape, b.shape)
    except ValueError:
        raise ValueError(f"operands could not be broadcast together with shapes {a.shape} {b.shape}") from None
    return broadcast_value(a, shape), broadcast_value(b, shape)


# --------------------------------------------------------------------------- elementwise
def _binary(opcode: str, x, y, dtype=None) -> Tensor:
    out_dt = np.dtype(dtype) if dtype is not None else find_common_type(x, y)
    out_dt = sanitize_dtype(out_dt)
    a, b = broadcast_pair(as_value(x, out_dt), as_value(y, out_dt))
    return wrap(G().op(opcode, a, b))


def add(x, y, dtype=None): return _binary("add", x, y, dtype)
def subtract(x, y, dtype=None): return _binary("sub", x, y, dtype)
def multiply(x, y, dtype=None): return _binary("mul", x, y, dtype)
def maximum(x, y, dtype=None): return _binary("max", x, y, dtype)
def minimum(x, y, dtype=None): return _binary("min", x, y, dtype)


def divide(x, y, dtype=None):
    if dtype is None:
        dt = find_common_type(x, y)
        if not is_float(dt):
            dtype = np.float32          # true division of integers yields a float, as in NumPy
    return _binary("div", x, y, dtype)


def power(x, y, dtype=None):
    return _binary("pow", x, y, dtype)


def _bitwise(opcode, x, y):
    dt = find_common_type(x, y)
    if is_float(dt):
        raise TypeError(f"bitwise {opcode} is not defined for {dt}")
    return _binary(opcode, x, y, dt)


def bitwise_and(x, y): return _bitwise("and", x, y)
def bitwise_or(x, y): return _bitwise("or", x, y)
def bitwise_xor(x, y): return _bitwise("xor", x, y)


def _compare(direction, x, y) -> Tensor:
    dt = sanitize_dtype(find_common_type(x, y))
    a, b = broadcast_pair(as_value(x, dt), as_value(y, dt))
    return wrap(G().op("compare", a, b, direction=direction))


def equal(x, y): return _compare("EQ", x, y)
def not_equal(x, y): return _compare("NE", x, y)
def greater(x, y): return _compare("GT", x, y)
def greater_equal(x, y): return _compare("GE", x, y)
def less(x, y): return _compare("LT", x, y)
def less_equal(x, y): return _compare("LE", x, y)


def _truth(x) -> Value:
    v = as_value(x)
    if v.dtype == np.bool_:
        return v
    zero = broadcast_value(as_value(0, v.dtype), v.shape)
    return G().op("compare", v, zero, direction="NE")


def _logical(opcode, x, y) -> Tensor:
    a, b = broadcast_pair(_truth(x), _truth(y))
    return wrap(G().op(opcode, a, b))


def logical_and(x, y): return _logical("and", x, y)
def logical_or(x, y): return _logical("or", x, y)
def logical_xor(x, y): return _logical("xor", x, y)


def _float_input(x) -> Value:
    v = as_value(x)
    if not is_float(v.dtype):
        v = convert(v, np.float32)
    return v


def _unary(opcode, x, float_only=True, dtype=None) -> Tensor:
    v = _float_input(x) if float_only else as_value(x)
    out = G().op(opcode, v)
    if dtype is not None:
        out = convert(out, dtype)
    return wrap(out)


def exp(x, dtype=None): return _unary("exp", x, dtype=dtype)
def log(x, dtype=None): return _unary("log", x, dtype=dtype)
def sqrt(x, dtype=None): return _unary("sqrt", x, dtype=dtype)
def sin(x, dtype=None): return _unary("sin", x, dtype=dtype)
def cos(x, dtype=None): return _unary("cos", x, dtype=dtype)
def tanh(x, dtype=None): return _unary("tanh", x, dtype=dtype)
def erf(x, dtype=None): return _unary("erf", x, dtype=dtype)
def rsqrt(x, dtype=None): return _unary("rsqrt", x, dtype=dtype)
def ceil(x, dtype=None): return _unary("ceil", x, dtype=dtype)
def floor(x, dtype=None): return _unary("floor", x, dtype=dtype)
def rint(x, dtype=None): return _unary("round_even", x, dtype=dtype)
def abs_(x, dtype=None): return _unary("abs", x, float_only=False, dtype=dtype)
def negative(x, dtype=None): return _unary("neg", x, float_only=False, dtype=dtype)
def sign(x, dtype=None): return _unary("sign", x, float_only=False, dtype=dtype)
def isfinite(x): return _unary("is_finite", x)


def arctan(x, dtype=None):
    v = _float_input(x)
    one = broadcast_value(as_value(1.0, v.dtype), v.shape)
    out = G().op("atan2", v, one)
    return wrap(convert(out, dtype) if dtype is not None else out)


def invert(x):
    v = as_value(x)
    if is_float(v.dtype):
        raise TypeError("invert is not defined for floating-point tensors")
    return wrap(G().op("not", v))


def logical_not(x):
    return wrap(G().op("not", _truth(x)))


def astype(x, dtype):
    v = as_value(x)
    dt = sanitize_dtype(np.dtype(dtype))
    if v.dtype == dt:
        return wrap(G().op("copy", v))
    return wrap(convert(v, dt))


def copy(x):
    return wrap(G().op("copy", as_value(x)))


def where(cond, x, y):
    dt = sanitize_dtype(find_common_type(x, y))
    c, a, b = _truth(cond), as_value(x, dt), as_value(y, dt)
    shape = np.broadcast_shapes(c.shape, a.shape, b.shape)
    return wrap(G().op("select", broadcast_value(c, shape), broadcast_value(a, shape), broadcast_value(b, shape)))


# --------------------------------------------------------------------------- reductions
def _norm_axes(axis, ndim) -> List[int]:
    if axis is None:
        return list(range(ndim))
    if isinstance(axis, (int, np.integer)):
        axis = (int(axis),)
    out = []
    for a in axis:
        a = int(a)
        if a < -ndim or a >= ndim:
            raise np.exceptions.AxisError(a, ndim)
        out.append(a % ndim)
    if len(set(out)) != len(out):
        raise ValueError("duplicate value in 'axis'")
    return sorted(out)


def _reduce(kind, x, axis=None, keepdims=False, dtype=None, **_ignored) -> Tensor:
    v = as_value(x)
    if v.dtype == np.bool_ and kind in ("sum", "prod"):
        v = convert(v, np.int32)
    axes = _norm_axes(axis, len(v.shape))
    out = G().op("reduce", v, kind=kind, axes=axes)
    if keepdims:
        shape = [1 if i in axes else d for i, d in enumerate(v.shape)]
        out = G().op("reshape", out, shape=shape)
    return wrap(out)


def sum_(x, axis=None, dtype=None, keepdims=False, **kw): return _reduce("sum", x, axis, keepdims)
def max_(x, axis=None, keepdims=False, **kw): return _reduce("max", x, axis, keepdims)
def min_(x, axis=None, keepdims=False, **kw): return _reduce("min", x, axis, keepdims)
def prod(x, axis=None, dtype=None, keepdims=False, **kw): return _reduce("prod", x, axis, keepdims)


def any_(x, axis=None, keepdims=False, **kw):
    v = _truth(x)
    axes = _norm_axes(axis, len(v.shape))
    out = G().op("reduce", v, kind="or", axes=axes)
    if keepdims:
        out = G().op("reshape", out, shape=[1 if i in axes else d for i, d in enumerate(v.shape)])
    return wrap(out)


def all_(x, axis=None, keepdims=False, **kw):
    v = _truth(x)
    axes = _norm_axes(axis, len(v.shape))
    out = G().op("reduce", v, kind="and", axes=axes)
    if keepdims:
        out = G().op("reshape", out, shape=[1 if i in axes else d for i, d in enumerate(v.shape)])
    return wrap(out)


def _arg_extreme(kind, x, axis=None, keepdims=False) -> Tensor:
    v = as_value(x)
    g = G()
    orig_shape = v.shape
    if axis is None:
        v = g.op("reshape", v, shape=[int(np.prod(v.shape, dtype=np.int64))])
        ax = 0
    else:
        ax = _norm_axes(axis, len(v.shape))[0]
    n = v.shape[ax]
    best = g.op("reduce", v, kind=kind, axes=[ax])
    kept = [1 if i == ax else d for i, d in enumerate(v.shape)]
    best_b = broadcast_value(g.op("reshape", best, shape=kept), v.shape)
    mask = g.op("compare", v, best_b, direction="EQ")
    iota = g.op("iota", shape=list(v.shape), dim=ax, dtype="i32")
    big = broadcast_value(as_value(n, np.int32), v.shape)
    cand = g.op("select", mask, iota, big)
    idx = g.op("reduce", cand, kind="min", axes=[ax])          # first occurrence
    if keepdims:
        shape = [1] * len(orig_shape) if axis is None else kept
        idx = g.op("reshape", idx, shape=shape)
    return wrap(idx)


def argmax(x, axis=None, keepdims=False, **kw): return _arg_extreme("max", x, axis, keepdims)
def argmin(x, axis=None, keepdims=False, **kw): return _arg_extreme("min", x, axis, keepdims)


# --------------------------------------------------------------------------- linalg
def matmul(x, y, dtype=None):
    dt = sanitize_dtype(np.dtype(dtype) if dtype is not None else find_common_type(x, y))
    a, b = as_value(x, dt), as_value(y, dt)
    g = G()
    if len(a.shape) == 0 or len(b.shape) == 0:
        raise ValueError("matmul: Input operand does not have enough dimensions")
    a1, b1 = len(a.shape) == 1, len(b.shape) == 1
    if a1:
        a = g.op("reshape", a, shape=[1, a.shape[0]])
    if b1:
        b = g.op("reshape", b, shape=[b.shape[0], 1])
    if a.shape[-1] != b.shape[-2]:
        raise ValueError(f"matmul: Input operand 1 has a mismatch in its core dimension 0 "
                         f"(size {b.shape[-2]} is different from {a.shape[-1]})")
    ba, bb = a.shape[:-2], b.shape[:-2]
    batch = np.broadcast_shapes(ba, bb)
    if ba != tuple(batch):
        a = broadcast_value(a, tuple(batch) + a.shape[-2:])
    if bb != tuple(batch):
        b = broadcast_value(b, tuple(batch) + b.shape[-2:])
    nb = len(batch)
    out = g.op("dot", a, b, lhs_batch=list(range(nb)), rhs_batch=list(range(nb)), lhs_contract=[nb + 1],
               rhs_contract=[nb])
    shape = list(out.shape)
    if a1:
        shape.pop(-2)
    if b1:
        shape.pop(-1)
    if tuple(shape) != out.shape:
        out = g.op("reshape", out, shape=shape)
    return wrap(out)


def dot(x, y):
    dt = sanitize_dtype(find_common_type(x, y))
    a, b = as_value(x, dt), as_value(y, dt)
    if len(a.shape) == 0 or len(b.shape) == 0:
        return multiply(x, y)
    rc = 0 if len(b.shape) == 1 else len(b.shape) - 2
    if a.shape[-1] != b.shape[rc]:
        raise ValueError(f"shapes {a.shape} and {b.shape} not aligned")
    return wrap(G().op("dot", a, b, lhs_batch=[], rhs_batch=[], lhs_contract=[len(a.shape) - 1], rhs_contract=[rc]))


# --------------------------------------------------------------------------- creation
def constant(value, dtype=None):
    if is_tensor(value):
        return astype(value, dtype) if dtype is not None else value
    if isinstance(value, (list, tuple)):
        value = np.asarray(value)
    if isinstance(value, np.ndarray):
        v = const(value)
        return wrap(convert(v, dtype) if dtype is not None else v)
    return wrap(as_value(value, dtype))


def _shape_tuple(shape) -> Tuple[int, ...]:
    if isinstance(shape, (int, np.integer)):
        return (int(shape),)
    return tuple(int(s) for s in shape)


def full(shape, fill_value, dtype=None):
    shape = _shape_tuple(shape)
    if is_tensor(fill_value):
        v = as_value(fill_value, dtype)
    else:
        dt = np.dtype(dtype) if dtype is not None else concrete(weak_type_of(fill_value))
        v = as_value(fill_value, sanitize_dtype(dt))
    return wrap(broadcast_value(v, shape) if shape else v)


def zeros(shape, dtype=np.float32): return full(shape, 0, dtype)
def ones(shape, dtype=np.float32): return full(shape, 1, dtype)


def full_like(x, fill_value, dtype=None, shape=None):
    dt = np.dtype(dtype) if dtype is not None else (x.dtype if hasattr(x, "dtype") else None)
    return full(shape if shape is not None else shape_of(x), fill_value, dt)


def zeros_like(x, dtype=None, shape=None): return full_like(x, 0, dtype, shape)
def ones_like(x, dtype=None, shape=None): return full_like(x, 1, dtype, shape)
def empty_like(x, dtype=None, shape=None): return full_like(x, 0, dtype, shape)


def _iota2(shape, dim):
    return G().op("iota", shape=list(shape), dim=dim, dtype="i32")


def _tri(x, k, lower: bool):
    v = as_value(x)
    if len(v.shape) < 2:
        raise ValueError("tril / triu need at least two dimensions")
    g = G()
    r = _iota2(v.shape, len(v.shape) - 2)
    c = _iota2(v.shape, len(v.shape) - 1)
    kk = broadcast_value(as_value(int(k), np.int32), v.shape)
    rk = g.op("add", r, kk)
    mask = g.op("compare", c, rk, direction="LE" if lower else "GE")
    zero = broadcast_value(as_value(0, v.dtype), v.shape)
    return wrap(g.op("select", mask, v, zero))


def tril(x, k=0): return _tri(x, k, True)
def triu(x, k=0): return _tri(x, k, False)


def diag(v, k=0):
    x = as_value(v)
    g = G()
    k = int(k)
    if len(x.shape) == 1:
        n = x.shape[0] + abs(k)
        r, c = _iota2((n, n), 0), _iota2((n, n), 1)
        kk = broadcast_value(as_value(k, np.int32), (n, n))
        mask = g.op("compare", c, g.op("add", r, kk), direction="EQ")
        # value for position (r, c) on the diagonal is x[min(r, c)]
        src = g.op("min", r, c)
        gathered = g.op("take", x, g.op("reshape", src, shape=[n * n]), axis=0)
        vals = g.op("reshape", gathered, shape=[n, n])
        zero = broadcast_value(as_value(0, x.dtype), (n, n))
        return wrap(g.op("select", mask, vals, zero))
    if len(x.shape) == 2:
        rows, cols = x.shape
        if k >= 0:
            length = max(0, min(rows, cols - k))
            r0, c0 = 0, k
        else:
            length = max(0, min(rows + k, cols))
            r0, c0 = -k, 0
        if length == 0:
            return wrap(const(np.zeros((0,), dtype=x.dtype)))
        flat = g.op("reshape", x, shape=[rows * cols])
        idx = np.arange(length, dtype=np.int32) * (cols + 1) + (r0 * cols + c0)
        return wrap(g.op("take", flat, const(idx), axis=0))
    raise ValueError("Input must be 1- or 2-d.")


# --------------------------------------------------------------------------- transforms
def reshape(x, shape, **kw):
    v = as_value(x)
    shape = list(_shape_tuple(shape))
    if shape.count(-1) > 1:
        raise ValueError("can only specify one unknown dimension")
    total = int(np.prod(v.shape, dtype=np.int64))
    if -1 in shape:
        known = int(np.prod([s for s in shape if s != -1], dtype=np.int64))
        if known == 0 or total % known:
            raise ValueError(f"cannot reshape array of size {total} into shape {tuple(shape)}")
        shape[shape.index(-1)] = total // known
    if int(np.prod(shape, dtype=np.int64)) != total:
        raise ValueError(f"cannot reshape array of size {total} into shape {tuple(shape)}")
    return wrap(G().op("reshape", v, shape=shape))


def transpose(x, axes=None):
    v = as_value(x)
    nd = len(v.shape)
    if axes is None:
        perm = list(range(nd - 1, -1, -1))
    else:
        axes = list(axes)
        if len(axes) != nd:
            raise ValueError("axes don't match array")
        perm = []
        for a in axes:
            a = int(a)
            if a < -nd or a >= nd:
                raise np.exceptions.AxisError(a, nd)
            perm.append(a % nd)
        if len(set(perm)) != nd:
            raise ValueError("repeated axis in transpose")
    return wrap(G().op("transpose", v, perm=perm))


def swapaxes(x, a, b):
    nd = len(shape_of(x))
    perm = list(range(nd))
    a, b = a % nd, b % nd
    perm[a], perm[b] = perm[b], perm[a]
    return transpose(x, perm)


def expand_dims(x, axis):
    v = as_value(x)
    axes = [axis] if isinstance(axis, (int, np.integer)) else list(axis)
    nd = len(v.shape) + len(axes)
    norm = []
    for a in axes:
        a = int(a)
        if a < -nd or a >= nd:
            raise np.exceptions.AxisError(a, nd)
        norm.append(a % nd)
    if len(set(norm)) != len(norm):
        raise ValueError("repeated axis")
    shape, it = [], iter(v.shape)
    for i in range(nd):
        shape.append(1 if i in norm else next(it))
    return wrap(G().op("reshape", v, shape=shape))


def squeeze(x, axis=None):
    v = as_value(x)
    nd = len(v.shape)
    if axis is None:
        drop = [i for i, d in enumerate(v.shape) if d == 1]
    else:
        drop = _norm_axes(axis, nd)
        for a in drop:
            if v.shape[a] != 1:
                raise ValueError("cannot select an axis to squeeze out which has size not equal to one")
    if not drop:
        return x if is_tensor(x) else wrap(v)
    return wrap(G().op("reshape", v, shape=[d for i, d in enumerate(v.shape) if i not in drop]))


def concatenate(arrays, axis=0, dtype=None, **kw):
    arrays = list(arrays)
    if not arrays:
        raise ValueError("need at least one array to concatenate")
    dts = [a.dtype if hasattr(a, "dtype") else np.asarray(a).dtype for a in arrays]
    dt = sanitize_dtype(np.dtype(dtype) if dtype is not None else np.result_type(*dts))
    vals = [as_value(a, dt) for a in arrays]
    if axis is None:
        vals = [G().op("reshape", v, shape=[int(np.prod(v.shape, dtype=np.int64))]) for v in vals]
        axis = 0
    nd = len(vals[0].shape)
    if axis < -nd or axis >= nd:
        raise np.exceptions.AxisError(axis, nd)
    axis %= nd
    if len(vals) == 1:
        return wrap(G().op("copy", vals[0]))
    return wrap(G().op("concat", *vals, axis=axis))


def stack(arrays, axis=0, **kw):
    arrays = list(arrays)
    nd = len(shape_of(arrays[0])) + 1
    if axis < -nd or axis >= nd:
        raise np.exceptions.AxisError(axis, nd)
    return concatenate([expand_dims(a, axis % nd) for a in arrays], axis=axis % nd)


def split(x, indices_or_sections, axis=0):
    v = as_value(x)
    nd = len(v.shape)
    axis = _norm_axes(axis, nd)[0]
    n = v.shape[axis]
    if isinstance(indices_or_sections, (int, np.integer)):
        k = int(indices_or_sections)
        if n % k:
            raise ValueError("array split does not result in an equal division")
        bounds = [i * (n // k) for i in range(k + 1)]
    else:
        bounds = [0] + [int(i) for i in indices_or_sections] + [n]
    out = []
    for s, e in zip(bounds[:-1], bounds[1:]):
        s, e = max(0, min(s, n)), max(0, min(e, n))
        e = max(s, e)
        start = [0] * nd
        limit = list(v.shape)
        start[axis], limit[axis] = s, e
        out.append(wrap(G().op("slice", v, start=start, limit=limit, stride=[1] * nd)))
    return out


def broadcast_to(x, shape, **kw):
    v = as_value(x)
    shape = _shape_tuple(shape)
    if v.shape == shape:
        return wrap(G().op("copy", v))
    return wrap(broadcast_value(v, shape))


def repeat(x, repeats, axis=None):
    if not isinstance(repeats, (int, np.integer)):
        raise TypeError("repeat needs a compile-time integer number of repeats")
    r = int(repeats)
    v = as_value(x)
    g = G()
    if axis is None:
        v = g.op("reshape", v, shape=[int(np.prod(v.shape, dtype=np.int64))])
        axis = 0
    nd = len(v.shape)
    axis = _norm_axes(axis, nd)[0]
    shape = list(v.shape)
    ex = shape[:axis + 1] + [1] + shape[axis + 1:]
    tgt = shape[:axis + 1] + [r] + shape[axis + 1:]
    t = g.op("reshape", v, shape=ex)
    t = g.op("broadcast", t, shape=tgt, dims=list(range(len(tgt))))
    shape[axis] *= r
    return wrap(g.op("reshape", t, shape=shape))


def tile(x, reps):
    v = as_value(x)
    reps = (int(reps),) if isinstance(reps, (int, np.integer)) else tuple(int(r) for r in reps)
    nd = max(len(v.shape), len(reps))
    shape = (1,) * (nd - len(v.shape)) + tuple(v.shape)
    reps = (1,) * (nd - len(reps)) + reps
    g = G()
    ex, tgt, out = [], [], []
    for d, r in zip(shape, reps):
        ex += [1, d]
        tgt += [r, d]
        out.append(r * d)
    t = g.op("reshape", v, shape=ex)
    t = g.op("broadcast", t, shape=tgt, dims=list(range(len(tgt))))
    return wrap(g.op("reshape", t, shape=out))


def flip(x, axis=None):
    v = as_value(x)
    nd = len(v.shape)
    axes = list(range(nd)) if axis is None else _norm_axes(axis, nd)
    g = G()
    for a in axes:
        idx = const(np.arange(v.shape[a] - 1, -1, -1, dtype=np.int32))
        v = g.op("take", v, idx, axis=a)
    return wrap(v)


def roll(x, shift, axis=None):
    v = as_value(x)
    g = G()
    if axis is None:
        flat = g.op("reshape", v, shape=[int(np.prod(v.shape, dtype=np.int64))])
        if not isinstance(shift, (int, np.integer)):
            raise ValueError("roll with axis=None needs a scalar shift")
        out = _roll_axis(flat, int(shift), 0)
        return wrap(g.op("reshape", out, shape=list(v.shape)))
    shifts = (shift,) if isinstance(shift, (int, np.integer)) else tuple(shift)
    axes = (axis,) if isinstance(axis, (int, np.integer)) else tuple(axis)
    try:
        pairs = np.broadcast(shifts, axes)
    except ValueError:
        raise ValueError("'shift' and 'axis' should be scalars or 1D sequences") from None
    for s, a in pairs:
        v = _roll_axis(v, int(s), _norm_axes(int(a), len(v.shape))[0])
    return wrap(v)


def _roll_axis(v: Value, shift: int, axis: int) -> Value:
    n = v.shape[axis]
    if n == 0 or shift % n == 0:
        return v
    idx = const(((np.arange(n) - shift) % n).astype(np.int32))
    return G().op("take", v, idx, axis=axis)


def pad(x, pad_width, mode="constant", constant_values=0, **kw):
    v = as_value(x)
    nd = len(v.shape)
    pw = np.asarray(pad_width)
    if pw.ndim == 0:
        pw = np.broadcast_to(pw, (nd, 2))
    elif pw.ndim == 1:
        pw = np.broadcast_to(pw.reshape(1, -1) if pw.size == 2 else pw.reshape(-1, 1), (nd, 2))
    pw = np.broadcast_to(pw, (nd, 2)).astype(int)
    g = G()
    if mode == "constant":
        pv = as_value(constant_values, v.dtype)
        if len(pv.shape):
            raise NotImplementedError("per-axis constant_values are not supported")
        return wrap(g.op("pad", v, pv, low=[int(p[0]) for p in pw], high=[int(p[1]) for p in pw]))
    if mode == "edge":
        for ax in range(nd):
            lo, hi = int(pw[ax][0]), int(pw[ax][1])
            if lo == 0 and hi == 0:
                continue
            n = v.shape[ax]
            idx = np.concatenate([np.zeros(lo, dtype=np.int32), np.arange(n, dtype=np.int32),
                                  np.full(hi, n - 1, dtype=np.int32)])
            v = g.op("take", v, const(idx), axis=ax)
        return wrap(v)
    raise NotImplementedError(f"pad mode {mode!r} is not supported (constant and edge are)")


# --------------------------------------------------------------------------- indexing
def _index_value(indices, dim: int) -> Value:
    """int32 index operand; constant negative indices are wrapped, dynamic ones are left to the op."""
    if is_tensor(indices):
        v = indices.backend_tensor
        return convert(v, np.int32) if v.dtype != np.int32 else v
    arr = np.asarray(indices)
    if arr.dtype.kind not in "iu":
        raise IndexError("indices must be integers")
    arr = arr.astype(np.int64)
    arr = np.where(arr < 0, arr + dim, arr)
    return const(arr.astype(np.int32))


def take(x, indices, axis=None, **kw):
    v = as_value(x)
    g = G()
    if axis is None:
        v = g.op("reshape", v, shape=[int(np.prod(v.shape, dtype=np.int64))])
        axis = 0
    axis = _norm_axes(axis, len(v.shape))[0]
    return wrap(g.op("take", v, _index_value(indices, v.shape[axis]), axis=axis))


def take_along_axis(x, indices, axis):
    v = as_value(x)
    g = G()
    if axis is None:
        v = g.op("reshape", v, shape=[int(np.prod(v.shape, dtype=np.int64))])
        axis = 0
    axis = _norm_axes(axis, len(v.shape))[0]
    idx = _index_value(indices, v.shape[axis])
    if len(idx.shape) != len(v.shape):
        raise ValueError("`indices` and `arr` must have the same number of dimensions")
    tgt = list(np.broadcast_shapes(tuple(1 if i == axis else d for i, d in enumerate(v.shape)),
                                   tuple(idx.shape)))
    tgt[axis] = idx.shape[axis]
    idx = broadcast_value(idx, tgt)
    xs = list(tgt)
    xs[axis] = v.shape[axis]
    v = broadcast_value(v, xs)
    return wrap(g.op("take_along_axis", v, idx, axis=axis))


def put_along_axis(x, indices, values, axis):
    v = as_value(x)
    if axis is None:
        raise NotImplementedError("put_along_axis with axis=None is not supported")
    axis = _norm_axes(axis, len(v.shape))[0]
    idx = _index_value(indices, v.shape[axis])
    if len(idx.shape) != len(v.shape):
        raise ValueError("`indices` and `arr` must have the same number of dimensions")
    tgt = list(v.shape)
    tgt[axis] = idx.shape[axis]
    idx = broadcast_value(idx, tgt)
    upd = broadcast_value(as_value(values, v.dtype), tgt)
    return wrap(G().op("put_along_axis", v, idx, upd, axis=axis))


def scatter_along_axis(x, indices, values, axis):
    """``out = x.copy(); out[..., indices, ...] = values`` with 1-D (or scalar) indices on `axis`."""
    v = as_value(x)
    axis = _norm_axes(axis, len(v.shape))[0]
    idx = _index_value(indices, v.shape[axis])
    g = G()
    if len(idx.shape) == 0:
        upd_shape = [1 if i == axis else d for i, d in enumerate(v.shape)]
        val = as_value(values, v.dtype)
        want = [d for i, d in enumerate(v.shape) if i != axis]
        if tuple(val.shape) != tuple(upd_shape):
            val = broadcast_value(val, want) if tuple(val.shape) != tuple(want) else val
            val = g.op("reshape", val, shape=upd_shape)
        zero = as_value(0, np.int32)
        starts = [idx if i == axis else zero for i in range(len(v.shape))]
        return wrap(g.op("dynamic_update_slice", v, val, *starts))
    if len(idx.shape) != 1:
        raise NotImplementedError("index assignment needs a scalar or 1-D index tensor")
    tgt = list(v.shape)
    tgt[axis] = idx.shape[0]
    upd = broadcast_value(as_value(values, v.dtype), tgt)
    return wrap(g.op("scatter_along_axis", v, idx, upd, axis=axis))


def static_slice(x, start, limit, stride=None):
    v = as_value(x)
    nd = len(v.shape)
    stride = [1] * nd if stride is None else list(stride)
    return wrap(G().op("slice", v, start=[int(s) for s in start], limit=[int(l) for l in limit],
                       stride=[int(s) for s in stride]))


def dynamic_update_slice(x, value, starts, strides=None, sizes=None, squeezed=None):
    """``out = x.copy(); out[start : start + size * stride : stride] = value`` per axis (static starts)."""
    v = as_value(x)
    nd = len(v.shape)
    strides = [1] * nd if strides is None else [int(s) for s in strides]
    val = as_value(value, v.dtype)
    if sizes is None:
        sizes = list(val.shape)
    sizes = [int(s) for s in sizes]
    g = G()
    if squeezed is not None:
        natural = [s for s, sq in zip(sizes, squeezed) if not sq]
    else:
        natural = sizes
    if tuple(val.shape) != tuple(sizes):
        if tuple(val.shape) != tuple(natural):
            val = broadcast_value(val, natural)
        val = g.op("reshape", val, shape=sizes)
    if any(s == 0 for s in sizes):
        return wrap(g.op("copy", v))
    return wrap(g.op("update_slice", v, val, start=[int(s) for s in starts], stride=strides))


def scatter_strided(x, value, starts, strides, sizes):
    return dynamic_update_slice(x, value, starts, strides=strides, sizes=sizes)


# --------------------------------------------------------------------------- nn / conv
def softmax(x, axis=-1):
    """Softmax over the last axis as ONE node (one row kernel on the device); other axes use the composition."""
    v = as_value(x)
    nd = len(v.shape)
    if nd == 0 or axis not in (-1, nd - 1) or np.dtype(v.dtype).kind != "f":
        return NotImplemented
    return wrap(G().op("softmax", v))


def rms_norm(x, weight=None, eps=1e-6, axis=-1):
    """RMSNorm over the last axis (fp32 statistics, optional weight of the row's length) as one node."""
    v = as_value(x)
    nd = len(v.shape)
    if nd == 0 or axis not in (-1, nd - 1) or np.dtype(v.dtype).kind != "f":
        return NotImplemented
    ins = [v]
    if weight is not None:
        wv = as_value(weight)
        if tuple(wv.shape) != (v.shape[-1],):
            return NotImplemented
        ins.append(wv)
    return wrap(G().add_node("rms_norm", ins, {"eps": float(eps)})[0])


def topk(x, k, axis=-1, is_ascend=False):
    v = as_value(x)
    nd = len(v.shape)
    if axis not in (-1, nd - 1):
        raise NotImplementedError("topk is implemented for the last axis only")
    g = G()
    if is_ascend:
        vals, idx = g.add_node("topk", [g.op("neg", v)], {"k": int(k)})
        return wrap(g.op("neg", vals)), wrap(idx)
    vals, idx = g.add_node("topk", [v], {"k": int(k)})
    return wrap(vals), wrap(idx)


def _tuple_n(v, n):
    return [int(v)] * n if isinstance(v, (int, np.integer)) else [int(t) for t in v]


def _conv(x, weight, bias, stride, padding, dilation, groups, nsp):
    dt = sanitize_dtype(find_common_type(x, weight))
    xv, wv = as_value(x, dt), as_value(weight, dt)
    if len(xv.shape) != nsp + 2 or len(wv.shape) != nsp + 2:
        raise ValueError(f"conv{nsp}d expects {nsp + 2}-D input and weight")
    if xv.shape[1] != wv.shape[1] * groups:
        raise ValueError("input channels do not match weight channels x groups")
    ins = [xv, wv]
    if bias is not None:
        ins.append(as_value(bias, dt))
    return wrap(G().add_node("conv", ins, {"stride": _tuple_n(stride, nsp), "padding": _tuple_n(padding, nsp),
                                           "dilation": _tuple_n(dilation, nsp), "groups": int(groups)})[0])


def conv2d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    return _conv(x, weight, bias, stride, padding, dilation, groups, 2)


def conv3d(x, weight, bias=None, stride=1, padding=0, dilation=1, groups=1):
    return _conv(x, weight, bias, stride, padding, dilation, groups, 3)


# --------------------------------------------------------------------------- collectives
_REDUCE_NAMES = {np.add: "add", np.multiply: "multiply", np.maximum: "maximum", np.minimum: "minimum"}


def _groups(replica_groups):
    return [[int(r) for r in grp] for grp in replica_groups]


def all_gather(data, all_gather_dim, replica_groups, **kw):
    v = as_value(data)
    return wrap(G().op("all_gather", v, dim=_norm_axes(all_gather_dim, len(v.shape))[0],
                       replica_groups=_groups(replica_groups)))


def all_reduce(data, replica_groups, reduce_op=np.add, **kw):
    return wrap(G().op("all_reduce", as_value(data), op=_REDUCE_NAMES.get(reduce_op, "add"),
                       replica_groups=_groups(replica_groups)))


def reduce_scatter(data, reduce_scatter_dim, replica_groups, reduce_op=np.add, **kw):
    v = as_value(data)
    return wrap(G().op("reduce_scatter", v, dim=_norm_axes(reduce_scatter_dim, len(v.shape))[0],
                       op=_REDUCE_NAMES.get(reduce_op, "add"), replica_groups=_groups(replica_groups)))


def all_to_all(data, split_dimension, concat_dimension, replica_groups, **kw):
    v = as_value(data)
    nd = len(v.shape)
    return wrap(G().op("all_to_all", v, split_dim=_norm_axes(split_dimension, nd)[0],
                       concat_dim=_norm_axes(concat_dimension, nd)[0], replica_groups=_groups(replica_groups)))
