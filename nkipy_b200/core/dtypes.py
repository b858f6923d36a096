"""Element types and the weak-type promotion lattice of the tracing frontend.

Behaviour follows the reference's JAX-style table
(nkipy/src/nkipy/core/backend/hlo.py:1055-1388): Python scalars are *weak* — they
adopt the dtype of the array operand instead of widening it — bool defers to
everything, integer + float gives the float type, f16 + bf16 meets at f32, mixed
fp8 variants do not promote, and 64-bit inputs are narrowed to 32 bits when a
kernel is traced (nkipy/src/nkipy/core/trace.py:24-46).  The implementation here is
a small lattice walk instead of an enumerated table.
"""

from __future__ import annotations

import warnings
from typing import Any, Optional

import ml_dtypes
import numpy as np

bfloat16 = np.dtype(ml_dtypes.bfloat16)
float8_e5m2 = np.dtype(ml_dtypes.float8_e5m2)
float8_e4m3 = np.dtype(ml_dtypes.float8_e4m3fn)
float8_e4m3fn = float8_e4m3

_NAMES = {
    "pred": np.dtype(np.bool_),
    "i8": np.dtype(np.int8), "i16": np.dtype(np.int16), "i32": np.dtype(np.int32), "i64": np.dtype(np.int64),
    "u8": np.dtype(np.uint8), "u16": np.dtype(np.uint16), "u32": np.dtype(np.uint32), "u64": np.dtype(np.uint64),
    "f16": np.dtype(np.float16), "bf16": bfloat16, "f32": np.dtype(np.float32), "f64": np.dtype(np.float64),
    "f8e5m2": float8_e5m2, "f8e4m3": float8_e4m3,
}
_BY_DTYPE = {v: k for k, v in _NAMES.items()}


def dtype_name(dt) -> str:
    """Short IR name ("f32", "bf16", "pred", ...) of a numpy dtype."""
    dt = np.dtype(dt)
    try:
        return _BY_DTYPE[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


def dtype_from_name(name: str) -> np.dtype:
    try:
        return _NAMES[name]
    except KeyError:
        raise TypeError(f"unknown dtype name {name!r}") from None


def all_dtypes():
    return list(_NAMES.values())


class WeakInt:
    """Sentinel for a Python int operand."""


class WeakFloat:
    """Sentinel for a Python float operand."""


_FP8 = (float8_e5m2, float8_e4m3)
_FLOAT_RANK = {float8_e5m2: 0, float8_e4m3: 0, np.dtype(np.float16): 1, bfloat16: 1, np.dtype(np.float32): 2,
               np.dtype(np.float64): 3}


def is_bool(dt) -> bool:
    return dt is not WeakInt and dt is not WeakFloat and np.dtype(dt) == np.bool_


def is_float(dt) -> bool:
    if dt is WeakFloat:
        return True
    if dt is WeakInt:
        return False
    return np.dtype(dt) in _FLOAT_RANK


def is_int(dt) -> bool:
    if dt is WeakInt:
        return True
    if dt is WeakFloat:
        return False
    return np.dtype(dt).kind in "iu"


def promote_types(a, b):
    """Join of two (possibly weak) types.  Returns a numpy dtype, or a weak sentinel when both are weak."""
    if a is b:
        return a
    weak_a, weak_b = a in (WeakInt, WeakFloat), b in (WeakInt, WeakFloat)
    if weak_a and weak_b:
        return WeakFloat
    if weak_a:
        a, b, weak_a, weak_b = b, a, weak_b, weak_a
    a = np.dtype(a)
    if weak_b:
        if b is WeakInt:
            return np.dtype(np.int32) if a == np.bool_ else a
        if a in _FLOAT_RANK:
            return a
        return np.dtype(np.float32)
    b = np.dtype(b)
    if a == b:
        return a
    if a == np.bool_:
        return b
    if b == np.bool_:
        return a
    fa, fb = a in _FLOAT_RANK, b in _FLOAT_RANK
    if fa and fb:
        if a in _FP8 and b in _FP8:
            raise TypeError(f"no implicit promotion between {dtype_name(a)} and {dtype_name(b)}")
        ra, rb = _FLOAT_RANK[a], _FLOAT_RANK[b]
        if ra == rb:            # f16 with bf16
            return np.dtype(np.float32)
        return a if ra > rb else b
    if fa:
        return a
    if fb:
        return b
    # two integer types
    sa, sb = a.kind == "i", b.kind == "i"
    if sa == sb:
        return a if a.itemsize >= b.itemsize else b
    signed, unsigned = (a, b) if sa else (b, a)
    need = max(signed.itemsize, unsigned.itemsize * 2)
    if need > 8:
        return np.dtype(np.float32)
    return np.dtype(f"int{need * 8}")


def weak_type_of(value: Any):
    """Type lattice element of an operand: tensors / arrays are strong, Python scalars weak."""
    if isinstance(value, bool):
        return np.dtype(np.bool_)
    if isinstance(value, int):
        return WeakInt
    if isinstance(value, float):
        return WeakFloat
    dt = getattr(value, "dtype", None)
    if dt is None:
        raise TypeError(f"cannot take the type of {type(value).__name__}")
    return np.dtype(dt)


def concrete(dt) -> np.dtype:
    if dt is WeakInt:
        return np.dtype(np.int32)
    if dt is WeakFloat:
        return np.dtype(np.float32)
    return np.dtype(dt)


def find_common_type(x: Any, y: Any) -> np.dtype:
    """Result dtype of a binary operation between x and y (tensors, arrays or Python scalars)."""
    return concrete(promote_types(weak_type_of(x), weak_type_of(y)))


def scalar_dtype(value: Any, other_dtype: Optional[np.dtype] = None) -> np.dtype:
    """dtype a scalar operand takes next to a tensor of `other_dtype`."""
    if other_dtype is None:
        return concrete(weak_type_of(value))
    return concrete(promote_types(weak_type_of(value), np.dtype(other_dtype)))


_NARROW = {np.dtype(np.float64): np.dtype(np.float32), np.dtype(np.int64): np.dtype(np.int32),
           np.dtype(np.uint64): np.dtype(np.uint32)}


def sanitize_dtype(dt) -> np.dtype:
    """64-bit types are not carried on the device: f64 -> f32, i64 -> i32, u64 -> u32."""
    dt = np.dtype(dt)
    return _NARROW.get(dt, dt)


def sanitize_array(arr: np.ndarray, name: str = "") -> np.ndarray:
    target = _NARROW.get(arr.dtype)
    if target is None:
        return arr
    label = f" '{name}'" if name else ""
    warnings.warn(f"Input tensor{label} has dtype {arr.dtype}, which the device path does not carry; "
                  f"casting to {target}.", stacklevel=3)
    return arr.astype(target)


def finfo_min(dt) -> float:
    dt = np.dtype(dt)
    if dt in _FLOAT_RANK:
        return float(ml_dtypes.finfo(dt).min) if dt in (bfloat16, *_FP8) else float(np.finfo(dt).min)
    if dt == np.bool_:
        return 0
    return int(np.iinfo(dt).min)


def finfo_max(dt) -> float:
    dt = np.dtype(dt)
    if dt in _FLOAT_RANK:
        return float(ml_dtypes.finfo(dt).max) if dt in (bfloat16, *_FP8) else float(np.finfo(dt).max)
    if dt == np.bool_:
        return 1
    return int(np.iinfo(dt).max)
