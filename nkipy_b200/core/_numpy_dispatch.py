"""NumPy function -> frontend op table.

When a NumPy function or ufunc is applied to a traced tensor, NumPy hands the call
to `NKIPyTensorRef.__array_ufunc__` / `__array_function__`, which look the function
up here.  Same coverage as the reference table
(nkipy/src/nkipy/core/_numpy_dispatch.py:27-159); `arctan2` and `positive` stay
unsupported there and here.
"""

from __future__ import annotations

import numpy as np

from . import ops
from .tensor import _tensor_apis

_registered = False


def _put_along_axis_inplace(arr, indices, values, axis):
    """np.put_along_axis mutates `arr` and returns None: emulate by rebinding the traced ref."""
    new = ops.put_along_axis(arr, indices, values, axis)
    if hasattr(arr, "_rebind"):
        arr._rebind(new)
        return None
    np.copyto(arr, new)
    return None


def register_all_numpy_apis() -> None:
    global _registered
    if _registered:
        return
    _registered = True
    t = _tensor_apis
    t.update({
        # binary
        np.add: ops.add, np.subtract: ops.subtract, np.multiply: ops.multiply, np.divide: ops.divide,
        np.true_divide: ops.divide, np.power: ops.power, np.maximum: ops.maximum, np.minimum: ops.minimum,
        np.bitwise_and: ops.bitwise_and, np.bitwise_or: ops.bitwise_or, np.bitwise_xor: ops.bitwise_xor,
        np.logaddexp: ops.logaddexp, np.remainder: ops.remainder, np.mod: ops.remainder,
        np.floor_divide: ops.floor_divide, np.matmul: ops.matmul,
        # comparison / logical
        np.equal: ops.equal, np.not_equal: ops.not_equal, np.greater: ops.greater,
        np.greater_equal: ops.greater_equal, np.less: ops.less, np.less_equal: ops.less_equal,
        np.logical_and: ops.logical_and, np.logical_or: ops.logical_or, np.logical_xor: ops.logical_xor,
        np.logical_not: ops.logical_not,
        # unary
        np.abs: ops.abs, np.absolute: ops.abs, np.exp: ops.exp, np.log: ops.log, np.sqrt: ops.sqrt,
        np.square: ops.square, np.negative: ops.negative, np.reciprocal: ops.reciprocal, np.sin: ops.sin,
        np.cos: ops.cos, np.tan: ops.tan, np.arctan: ops.arctan, np.tanh: ops.tanh, np.ceil: ops.ceil,
        np.floor: ops.floor, np.rint: ops.rint, np.trunc: ops.trunc, np.sign: ops.sign, np.invert: ops.invert,
        np.bitwise_not: ops.bitwise_not, np.clip: ops.clip, np.log1p: ops.log1p, np.log2: ops.log2,
        np.expm1: ops.expm1, np.round: ops.round_, np.around: ops.round_, np.isnan: ops.isnan,
        np.isfinite: ops.isfinite,
        # reductions
        np.sum: ops.sum, np.max: ops.max, np.amax: ops.max, np.min: ops.min, np.amin: ops.min, np.mean: ops.mean,
        np.any: ops.any, np.all: ops.all, np.var: ops.var, np.std: ops.std, np.argmax: ops.argmax,
        np.argmin: ops.argmin, np.cumsum: ops.cumsum, np.prod: ops.prod, np.count_nonzero: ops.count_nonzero,
        # linalg
        np.dot: ops.dot, np.linalg.norm: ops.norm, np.outer: ops.outer, np.trace: ops.trace,
        # transforms
        np.reshape: ops.reshape, np.transpose: ops.transpose, np.expand_dims: ops.expand_dims,
        np.concatenate: ops.concatenate, np.split: ops.split, np.copy: ops.copy, np.repeat: ops.repeat,
        np.squeeze: ops.squeeze, np.pad: ops.pad, np.swapaxes: ops.swapaxes, np.stack: ops.stack, np.diff: ops.diff,
        np.flip: ops.flip, np.tile: ops.tile, np.roll: ops.roll, np.ravel: lambda x: ops.reshape(x, (-1,)),
        np.sort: lambda x, axis=-1, kind=None: ops.sort(x, axis=axis),
        np.argsort: lambda x, axis=-1, kind=None: ops.argsort(x, axis=axis),
        # creation
        np.zeros_like: ops.zeros_like, np.ones_like: ops.ones_like, np.empty_like: ops.empty_like,
        np.full_like: ops.full_like, np.tril: ops.tril, np.triu: ops.triu, np.diag: ops.diag,
        # indexing
        np.where: ops.where, np.take: ops.take, np.take_along_axis: ops.take_along_axis,
        np.put_along_axis: _put_along_axis_inplace,
        np.broadcast_to: ops.broadcast_to, np.copyto: ops.copyto,
    })
