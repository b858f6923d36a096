"""The traced tensor: what a kernel function sees instead of a NumPy array.

`NKIPyTensorRef` wraps an IR `Value`.  NumPy functions and ufuncs applied to it are
routed through ``__array_ufunc__`` / ``__array_function__`` to the op registry,
arithmetic dunders and the usual ndarray methods are provided, and indexing /
slice-assignment are lowered to IR ops.  Mutation (``x[...] = v``) is functional
underneath: the ref is rebound to a new value and, if it is a kernel parameter,
the parameter is marked mutated so the tracer can alias an output to it.

Same user-visible behaviour as the reference's tensor
(nkipy/src/nkipy/core/tensor.py:387-948): `__array__` refuses to materialise,
unregistered NumPy functions raise ``NotImplementedError``, at most boolean masks
are rejected as indices, `a[np.arange(N), idx]`-style multi-array indexing follows
NumPy's layout rules.
"""

from __future__ import annotations

import os
import sys
from typing import Any, List, Optional, Sequence, Tuple

import numpy as np

from .backend import set_source_location
from .ir import Value

_CORE_DIR = os.path.dirname(os.path.abspath(__file__))
_tensor_apis = {}   # numpy function / ufunc -> implementation, filled by _numpy_dispatch


def find_source_loc() -> Optional[Tuple[str, int]]:
    """(file, line) of the innermost frame outside this package: the user's kernel line."""
    f = sys._getframe(1)
    while f is not None:
        fn = f.f_code.co_filename
        if not os.path.abspath(fn).startswith(_CORE_DIR) and "numpy" not in fn.split(os.sep)[-3:]:
            return (fn, f.f_lineno)
        f = f.f_back
    return None


def _ops():
    from . import ops

    return ops


class TensorArithmeticMixin:
    def __add__(self, o): return _ops().add(self, o)
    def __radd__(self, o): return _ops().add(o, self)
    def __sub__(self, o): return _ops().subtract(self, o)
    def __rsub__(self, o): return _ops().subtract(o, self)
    def __mul__(self, o): return _ops().multiply(self, o)
    def __rmul__(self, o): return _ops().multiply(o, self)
    def __truediv__(self, o): return _ops().divide(self, o)
    def __rtruediv__(self, o): return _ops().divide(o, self)
    def __floordiv__(self, o): return _ops().floor_divide(self, o)
    def __rfloordiv__(self, o): return _ops().floor_divide(o, self)
    def __mod__(self, o): return _ops().remainder(self, o)
    def __rmod__(self, o): return _ops().remainder(o, self)
    def __pow__(self, o): return _ops().power(self, o)
    def __rpow__(self, o): return _ops().power(o, self)
    def __matmul__(self, o): return _ops().matmul(self, o)
    def __rmatmul__(self, o): return _ops().matmul(o, self)
    def __neg__(self): return _ops().negative(self)
    def __pos__(self): return self
    def __abs__(self): return _ops().abs(self)
    def __invert__(self): return _ops().invert(self)
    def __and__(self, o): return _ops().bitwise_and(self, o)
    def __rand__(self, o): return _ops().bitwise_and(o, self)
    def __or__(self, o): return _ops().bitwise_or(self, o)
    def __ror__(self, o): return _ops().bitwise_or(o, self)
    def __xor__(self, o): return _ops().bitwise_xor(self, o)
    def __rxor__(self, o): return _ops().bitwise_xor(o, self)
    def __lt__(self, o): return _ops().less(self, o)
    def __le__(self, o): return _ops().less_equal(self, o)
    def __gt__(self, o): return _ops().greater(self, o)
    def __ge__(self, o): return _ops().greater_equal(self, o)
    def __eq__(self, o): return _ops().equal(self, o)
    def __ne__(self, o): return _ops().not_equal(self, o)
    # in-place operators are functional: Python rebinds the name, the parameter is not mutated
    def __iadd__(self, o): return _ops().add(self, o)
    def __isub__(self, o): return _ops().subtract(self, o)
    def __imul__(self, o): return _ops().multiply(self, o)
    def __itruediv__(self, o): return _ops().divide(self, o)
    def __ifloordiv__(self, o): return _ops().floor_divide(self, o)
    def __imod__(self, o): return _ops().remainder(self, o)
    def __ipow__(self, o): return _ops().power(self, o)
    def __imatmul__(self, o): return _ops().matmul(self, o)
    def __iand__(self, o): return _ops().bitwise_and(self, o)
    def __ior__(self, o): return _ops().bitwise_or(self, o)
    def __ixor__(self, o): return _ops().bitwise_xor(self, o)
    __hash__ = object.__hash__


class TensorOperationMixin:
    def transpose(self, *axes):
        if len(axes) == 1 and isinstance(axes[0], (tuple, list)):
            axes = tuple(axes[0])
        return _ops().transpose(self, axes if axes else None)

    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        return _ops().reshape(self, shape)

    def astype(self, dtype): return _ops().astype(self, dtype)
    def mean(self, axis=None, dtype=None, keepdims=False): return _ops().mean(self, axis=axis, keepdims=keepdims)
    def sum(self, axis=None, dtype=None, keepdims=False): return _ops().sum(self, axis=axis, keepdims=keepdims)
    def prod(self, axis=None, dtype=None, keepdims=False): return _ops().prod(self, axis=axis, keepdims=keepdims)
    def var(self, axis=None, dtype=None, ddof=0, keepdims=False):
        return _ops().var(self, axis=axis, ddof=ddof, keepdims=keepdims)
    def std(self, axis=None, dtype=None, ddof=0, keepdims=False):
        return _ops().std(self, axis=axis, ddof=ddof, keepdims=keepdims)
    def squeeze(self, axis=None): return _ops().squeeze(self, axis=axis)
    def max(self, axis=None, keepdims=False): return _ops().max(self, axis=axis, keepdims=keepdims)
    def min(self, axis=None, keepdims=False): return _ops().min(self, axis=axis, keepdims=keepdims)
    def argmax(self, axis=None, keepdims=False): return _ops().argmax(self, axis=axis, keepdims=keepdims)
    def argmin(self, axis=None, keepdims=False): return _ops().argmin(self, axis=axis, keepdims=keepdims)
    def copy(self): return _ops().copy(self)
    def clip(self, min=None, max=None): return _ops().clip(self, min, max)
    def ravel(self): return _ops().reshape(self, (-1,))
    def flatten(self): return _ops().reshape(self, (-1,))
    def swapaxes(self, a, b): return _ops().swapaxes(self, a, b)
    def dot(self, other): return _ops().dot(self, other)


def _is_int(x) -> bool:
    return isinstance(x, (int, np.integer)) and not isinstance(x, (bool, np.bool_))


class NKIPyTensorRef(TensorArithmeticMixin, TensorOperationMixin):
    __slots__ = ("backend_tensor", "_shape", "_dtype", "_name", "_original_parameter", "_is_mutated")
    __array_priority__ = 1000

    def __init__(self, backend_tensor: Value, name: str = "", original_parameter: Optional[Value] = None):
        self.backend_tensor = backend_tensor
        self._shape = tuple(backend_tensor.shape)
        self._dtype = np.dtype(backend_tensor.dtype)
        self._name = name
        self._original_parameter = original_parameter
        self._is_mutated = False

    # ------------------------------------------------------------------ array protocol
    @property
    def shape(self): return tuple(self.backend_tensor.shape)
    @property
    def dtype(self): return np.dtype(self.backend_tensor.dtype)
    @property
    def ndim(self): return len(self.backend_tensor.shape)
    @property
    def size(self): return int(np.prod(self.shape, dtype=np.int64))
    @property
    def T(self): return _ops().transpose(self, None)
    @property
    def name(self): return self._name
    @property
    def strides(self):
        st, acc = [], self.dtype.itemsize
        for d in reversed(self.shape):
            st.append(acc)
            acc *= d
        return tuple(reversed(st))

    def __len__(self):
        if self.ndim == 0:
            raise TypeError("len() of unsized object")
        return self.shape[0]

    def __repr__(self):
        return f"NKIPyTensorRef(shape={self.shape}, dtype={self.dtype}, name={self._name!r})"

    def __array__(self, *args, **kwargs):
        raise TypeError("A traced tensor cannot be converted to a NumPy array: its value is not known at trace "
                        "time. Use NumPy functions on it instead, or pass concrete values as non-array arguments.")

    def __bool__(self):
        raise TypeError("The truth value of a traced tensor is not known at trace time; use np.where / np.select.")

    def __iter__(self):
        for i in range(len(self)):
            yield self[i]

    def __array_ufunc__(self, ufunc, method, *inputs, **kwargs):
        if method != "__call__":
            if method == "reduce":
                red = {np.add: "sum", np.maximum: "max", np.minimum: "min", np.multiply: "prod"}.get(ufunc)
                if red is not None:
                    set_source_location(find_source_loc())
                    return getattr(_ops(), red)(inputs[0], axis=kwargs.get("axis", 0),
                                                keepdims=kwargs.get("keepdims", False))
            raise NotImplementedError(f"ufunc method {ufunc.__name__}.{method} is not supported on traced tensors")
        impl = _tensor_apis.get(ufunc)
        if impl is None:
            raise NotImplementedError(f"NumPy function '{ufunc.__name__}' has not been implemented")
        kwargs.pop("out", None)
        set_source_location(find_source_loc())
        return impl(*inputs, **kwargs)

    def __array_function__(self, func, types, args, kwargs):
        impl = _tensor_apis.get(func)
        if impl is None:
            raise NotImplementedError(f"NumPy function '{func.__name__}' has not been implemented")
        set_source_location(find_source_loc())
        return impl(*args, **kwargs)

    # ------------------------------------------------------------------ indexing
    def _expand_key(self, key) -> List[Any]:
        if not isinstance(key, tuple):
            key = (key,)
        key = list(key)
        n_ell = sum(1 for k in key if k is Ellipsis)
        if n_ell > 1:
            raise IndexError("an index can only have a single ellipsis ('...')")
        consumed = sum(1 for k in key if k is not None and k is not Ellipsis)
        if consumed > self.ndim:
            raise IndexError(f"too many indices for tensor: tensor is {self.ndim}-dimensional, "
                             f"but {consumed} were indexed")
        fill = [slice(None)] * (self.ndim - consumed)
        if n_ell:
            i = key.index(Ellipsis)
            key[i:i + 1] = fill
        else:
            key.extend(fill)
        return key

    @staticmethod
    def _classify(k):
        if k is None:
            return "new"
        if isinstance(k, slice):
            return "slice"
        if _is_int(k):
            return "int"
        if isinstance(k, NKIPyTensorRef):
            if k.dtype == np.bool_:
                raise NotImplementedError("boolean mask indexing is not supported in traced kernels")
            return "tensor"
        if isinstance(k, (list, tuple, np.ndarray)):
            arr = np.asarray(k)
            if arr.dtype == np.bool_:
                raise NotImplementedError("boolean mask indexing is not supported in traced kernels")
            if arr.dtype.kind not in "iu":
                raise IndexError("arrays used as indices must be of integer type")
            return "array"
        if isinstance(k, (bool, np.bool_)):
            raise NotImplementedError("boolean indexing is not supported in traced kernels")
        raise IndexError(f"unsupported index type {type(k).__name__}")

    def __getitem__(self, key):
        ops = _ops()
        set_source_location(find_source_loc())
        key = self._expand_key(key)
        kinds = [self._classify(k) for k in key]
        has_adv = any(k in ("tensor", "array") for k in kinds)
        x = self
        # ---- pass 1: slices (and ints when no array index is present) as one static slice
        starts, limits, strides, flips = [], [], [], []
        dim = 0
        for k, kind in zip(key, kinds):
            if kind == "new":
                continue
            n = self.shape[dim]
            if kind == "slice":
                s, e, st = k.indices(n)
                if st > 0:
                    cnt = max(0, (e - s + st - 1) // st)
                    starts.append(s); limits.append(s + (cnt - 1) * st + 1 if cnt else s); strides.append(st)
                    flips.append(False)
                else:
                    cnt = max(0, (s - e - st - 1) // (-st))
                    last = s + (cnt - 1) * st if cnt else s
                    starts.append(last if cnt else s); limits.append(s + 1 if cnt else s); strides.append(-st)
                    flips.append(cnt > 1)
            elif kind == "int":
                i = int(k)
                if i < -n or i >= n:
                    raise IndexError(f"index {i} is out of bounds for axis {dim} with size {n}")
                i %= n
                starts.append(i); limits.append(i + 1); strides.append(1); flips.append(False)
            else:
                starts.append(0); limits.append(n); strides.append(1); flips.append(False)
            dim += 1
        if any(s != 0 or l != d or st != 1 for s, l, st, d in zip(starts, limits, strides, self.shape)):
            x = ops.static_slice(x, starts, limits, strides)
        for ax, fl in enumerate(flips):
            if fl:
                x = ops.flip(x, axis=ax)
        # ---- pass 2: advanced indices
        adv_axes = []          # axes of x consumed by advanced indices (ints count when arrays are present)
        adv_idx = []
        dim = 0
        positions = []         # position in the expanded key, to decide adjacency
        for pos, (k, kind) in enumerate(zip(key, kinds)):
            if kind == "new":
                continue
            if kind in ("tensor", "array") or (kind == "int" and has_adv):
                adv_axes.append(dim)
                positions.append(pos)
                if kind == "int":
                    adv_idx.append(np.zeros((), dtype=np.int32))     # already sliced to size 1
                elif kind == "array":
                    arr = np.asarray(k).astype(np.int64)
                    n = self.shape[dim]
                    if arr.size and (arr.min() < -n or arr.max() >= n):
                        raise IndexError(f"index out of bounds for axis {dim} with size {n}")
                    adv_idx.append(np.where(arr < 0, arr + n, arr).astype(np.int32))
                else:
                    adv_idx.append(k)
            dim += 1
        drop_int_axes = [] if has_adv else [i for i, kd in enumerate(k for k in kinds if k != "new") if kd == "int"]
        if has_adv:
            x = self._gather(x, adv_axes, adv_idx, positions, key, kinds)
            return x
        # ---- pass 3: drop int axes, insert new axes
        out_shape = []
        dim = 0
        for kind in kinds:
            if kind == "new":
                out_shape.append(1)
            else:
                if kind != "int":
                    out_shape.append(x.shape[dim])
                dim += 1
        if tuple(out_shape) != x.shape:
            x = ops.reshape(x, tuple(out_shape))
        elif x is self:
            x = ops.copy(x) if False else x
        return x

    def _gather(self, x, adv_axes, adv_idx, positions, key, kinds):
        """NumPy advanced indexing on `x` (already basic-sliced): advanced axes are moved to the
        front, flattened into one axis and gathered with a linear index."""
        ops = _ops()
        nd = x.ndim
        rest = [a for a in range(nd) if a not in adv_axes]
        # broadcast shape of the index operands
        shapes = [tuple(i.shape) for i in adv_idx]
        bshape = np.broadcast_shapes(*shapes) if shapes else ()
        if len(adv_axes) == 1 and not isinstance(adv_idx[0], np.ndarray) or len(adv_axes) == 1:
            idx = adv_idx[0]
            res = ops.take(x, idx, axis=adv_axes[0])
            first = adv_axes[0]
            idx_nd = len(np.shape(idx)) if not isinstance(idx, NKIPyTensorRef) else idx.ndim
            front = False
        else:
            perm = list(adv_axes) + rest
            xt = ops.transpose(x, perm) if perm != list(range(nd)) else x
            dims = [x.shape[a] for a in adv_axes]
            flat = int(np.prod(dims, dtype=np.int64))
            xt = ops.reshape(xt, (flat,) + tuple(x.shape[a] for a in rest))
            lin = None
            stride = 1
            for d, i in zip(reversed(dims), reversed(adv_idx)):
                term = i if stride == 1 else ops.multiply(i, np.int32(stride)) if isinstance(i, NKIPyTensorRef) \
                    else (np.asarray(i, dtype=np.int64) * stride).astype(np.int32)
                if lin is None:
                    lin = term
                elif isinstance(lin, np.ndarray) and isinstance(term, np.ndarray):
                    lin = (lin.astype(np.int64) + term).astype(np.int32)
                else:
                    lin = ops.add(term, lin) if isinstance(term, NKIPyTensorRef) else ops.add(lin, term)
                stride *= d
            if isinstance(lin, np.ndarray):
                lin = np.broadcast_to(lin, bshape).astype(np.int32)
            elif tuple(lin.shape) != tuple(bshape):
                lin = ops.broadcast_to(lin, bshape)
            res = ops.take(xt, lin, axis=0)            # bshape + rest dims
            first, idx_nd = 0, len(bshape)
            # NumPy: adjacent advanced indices keep their place, separated ones go first
            adjacent = all(b - a == 1 for a, b in zip(positions, positions[1:]))
            if adjacent and adv_axes[0] > 0:
                lead = adv_axes[0]                    # number of kept axes before the advanced block
                r = res.ndim
                perm2 = list(range(idx_nd, idx_nd + lead)) + list(range(idx_nd)) + list(range(idx_nd + lead, r))
                res = ops.transpose(res, perm2)
                first = lead
            front = not adjacent
        # new axes requested with None
        if any(k == "new" for k in kinds):
            out_shape = []
            # rebuild shape walking the key: advanced block contributes once at its place
            res_dims = list(res.shape)
            placed = False
            src = 0
            kept_before = 0
            shape_iter = []
            dim = 0
            for pos, kind in enumerate(kinds):
                if kind == "new":
                    shape_iter.append("new")
                elif kind in ("tensor", "array", "int"):
                    if not placed:
                        shape_iter.append("adv")
                        placed = True
                else:
                    shape_iter.append("keep")
            # only the simple case (no separated advanced indices) supports mixing with None
            if front:
                raise NotImplementedError("newaxis combined with separated advanced indices is not supported")
            cursor = 0
            for item in shape_iter:
                if item == "new":
                    out_shape.append(1)
                elif item == "adv":
                    out_shape.extend(res_dims[cursor:cursor + idx_nd])
                    cursor += idx_nd
                else:
                    out_shape.append(res_dims[cursor])
                    cursor += 1
            res = ops.reshape(res, tuple(out_shape))
        return res

    def __setitem__(self, key, value):
        ops = _ops()
        set_source_location(find_source_loc())
        key = self._expand_key(key)
        kinds = [self._classify(k) for k in key]
        if any(k == "new" for k in kinds):
            raise NotImplementedError("newaxis is not supported in slice assignment")
        adv = [i for i, k in enumerate(kinds) if k in ("tensor", "array")]
        if not adv:
            starts, strides, sizes, squeeze = [], [], [], []
            for ax, (k, kind) in enumerate(zip(key, kinds)):
                n = self.shape[ax]
                if kind == "int":
                    i = int(k)
                    if i < -n or i >= n:
                        raise IndexError(f"index {i} is out of bounds for axis {ax} with size {n}")
                    starts.append(i % n); strides.append(1); sizes.append(1); squeeze.append(True)
                else:
                    s, e, st = k.indices(n)
                    if st < 0:
                        raise NotImplementedError("negative-step slice assignment is not supported")
                    cnt = max(0, (e - s + st - 1) // st)
                    starts.append(s); strides.append(st); sizes.append(cnt); squeeze.append(False)
            new = ops.dynamic_update_slice(self, value, starts, strides=strides, sizes=sizes, squeezed=squeeze)
        elif len(adv) == 1:
            ax = adv[0]
            others_full = all(
                kinds[i] == "slice" and key[i].indices(self.shape[i]) == (0, self.shape[i], 1)
                for i in range(len(key)) if i != ax)
            idx = key[ax]
            if not others_full:
                raise NotImplementedError("index assignment supports one index tensor with full slices elsewhere")
            new = ops.scatter_along_axis(self, idx, value, axis=ax)
        else:
            raise NotImplementedError("assignment through several index tensors is not supported")
        self._rebind(new)

    def _rebind(self, new: "NKIPyTensorRef") -> None:
        """Emulate in-place mutation: this ref now denotes the updated value."""
        self.backend_tensor = new.backend_tensor
        self._is_mutated = True
