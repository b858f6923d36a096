"""Kernel specifications: what shapes, dtypes and scalar arguments a kernel accepts.

Specification files (``tests/kernels/*.py``) export a ``kernel_specs`` list; the spec-driven
integration test runs every kernel on its default inputs and the fuzz test on randomly drawn valid
ones, comparing direct mode against the traced graph (and the device where there is one).  The schema
is field-compatible with the reference's (nkipy/src/nkipy/core/specs.py:11-92): a file written against
either package imports against the other.  Added here: `sample` / `make` helpers that draw valid
shapes and build input arrays, so the tests need no per-kernel glue.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, List, Optional, Sequence, Tuple, Union

import numpy as np

Dim = Union[int, Tuple[Optional[int], Optional[int]], None]


@dataclass
class ShapeSpec:
    """Shape constraint, one entry per dimension: an int (exactly that size), ``(lo, hi)`` with either bound
    possibly None (a range), or None (any size).  `default` is the shape used when nothing else is asked."""

    dims: List[Dim]
    default: Tuple[int, ...]

    def is_valid(self, shape: Sequence[int]) -> bool:
        if len(shape) != len(self.dims):
            return False
        for want, have in zip(self.dims, shape):
            if want is None:
                continue
            if isinstance(want, (tuple, list)):
                lo, hi = want
                if (lo is not None and have < lo) or (hi is not None and have > hi):
                    return False
            elif int(want) != int(have):
                return False
        return True

    def sample(self, rng: np.random.Generator, free_range: Tuple[int, int] = (1, 48)) -> Tuple[int, ...]:
        """A random valid shape; unconstrained sizes are drawn from `free_range`."""
        out = []
        for want in self.dims:
            if want is None:
                lo, hi = free_range
            elif isinstance(want, (tuple, list)):
                lo = free_range[0] if want[0] is None else want[0]
                hi = max(lo, free_range[1]) if want[1] is None else want[1]
            else:
                out.append(int(want))
                continue
            out.append(int(rng.integers(lo, hi + 1)))
        return tuple(out)


@dataclass
class TypeSpec:
    """The dtypes an input accepts and the one used by default."""

    allowed: List[Any]
    default: Any

    def is_valid(self, dtype) -> bool:
        try:
            want = np.dtype(dtype)
        except TypeError:
            return dtype in self.allowed
        return any(np.dtype(a) == want for a in self.allowed)

    def sample(self, rng: np.random.Generator):
        return self.allowed[int(rng.integers(0, len(self.allowed)))]


@dataclass(kw_only=True)
class InputSpec:
    dtype_spec: TypeSpec
    description: str = ""
    default_value: Any = None


@dataclass(kw_only=True)
class ScalarInputSpec(InputSpec):
    """A compile-time scalar argument (a Python value baked into the trace)."""

    description: str = "Scalar input"

    def make(self, rng: Optional[np.random.Generator] = None, dtype=None):
        if self.default_value is not None:
            return self.default_value
        dt = np.dtype(dtype if dtype is not None else self.dtype_spec.default)
        return dt.type(1).item()


@dataclass(kw_only=True)
class TensorInputSpec(InputSpec):
    shape_spec: ShapeSpec
    description: str = "Tensor input"
    # optional builder (shape, dtype, rng) -> array for inputs that must not be plain noise (indices, masks)
    generator: Optional[Callable[[Tuple[int, ...], Any, np.random.Generator], np.ndarray]] = None

    def make(self, rng: Optional[np.random.Generator] = None, shape=None, dtype=None) -> np.ndarray:
        rng = rng or np.random.default_rng(0)
        if self.default_value is not None and shape is None and dtype is None:
            return np.array(self.default_value)
        shape = tuple(shape if shape is not None else self.shape_spec.default)
        dt = np.dtype(dtype if dtype is not None else self.dtype_spec.default)
        if self.generator is not None:
            return self.generator(shape, dt, rng)
        if dt.kind == "f":
            return rng.standard_normal(shape).astype(dt)
        if dt.kind == "b":
            return rng.random(shape) > 0.5
        return rng.integers(0, 8, shape).astype(dt)


@dataclass
class KernelSpec:
    """A kernel function with the specification of each of its inputs."""

    function: Any
    inputs: List[InputSpec]
    is_pure_numpy: bool = True
    description: str = ""

    def default_inputs(self, rng: Optional[np.random.Generator] = None) -> list:
        rng = rng or np.random.default_rng(0)
        return [i.make(rng) for i in self.inputs]

    def random_inputs(self, rng: np.random.Generator, same_shape: bool = True) -> list:
        """Valid random inputs.  With same_shape, tensor inputs whose constraints admit the first tensor's
        sampled shape share it (elementwise kernels need matching shapes)."""
        first_shape, dtype, out = None, None, []
        for spec in self.inputs:
            if isinstance(spec, TensorInputSpec):
                shape = spec.shape_spec.sample(rng)
                if same_shape and first_shape is not None and spec.shape_spec.is_valid(first_shape):
                    shape = first_shape
                if first_shape is None:
                    first_shape = shape
                if dtype is None or not spec.dtype_spec.is_valid(dtype):
                    dtype = spec.dtype_spec.sample(rng)
                out.append(spec.make(rng, shape, dtype))
            else:
                out.append(spec.make(rng))
        return out


class CommonTypes:
    FLOATS = TypeSpec(allowed=[np.float32, np.float16], default=np.float32)
    INTS = TypeSpec(allowed=[np.int8, np.int16, np.int32, np.int64], default=np.int32)
    BOOL = TypeSpec(allowed=[bool], default=bool)
