"""Kernel specifications that drive the spec-based integration and fuzz tests
(nkipy/src/nkipy/core/specs.py:11-92 in the reference)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, List, Optional, Sequence, Tuple

import numpy as np


@dataclass
class ShapeSpec:
    """Allowed shapes: per-dimension (min, max) ranges or fixed ints, plus a default shape."""
    dims: Sequence[Any]
    default: Tuple[int, ...]

    def is_valid(self, shape: Sequence[int]) -> bool:
        if len(shape) != len(self.dims):
            return False
        for d, s in zip(self.dims, shape):
            if d is None:
                continue
            if isinstance(d, (tuple, list)):
                lo, hi = d
                if not (lo <= s <= hi):
                    return False
            elif s != d:
                return False
        return True

    def sample(self, rng: np.random.Generator) -> Tuple[int, ...]:
        out = []
        for d, dflt in zip(self.dims, self.default):
            if d is None:
                out.append(dflt)
            elif isinstance(d, (tuple, list)):
                out.append(int(rng.integers(d[0], d[1] + 1)))
            else:
                out.append(int(d))
        return tuple(out)


@dataclass
class TypeSpec:
    allowed: Sequence[Any]
    default: Any = np.float32

    def is_valid(self, dtype) -> bool:
        return np.dtype(dtype) in [np.dtype(a) for a in self.allowed]


class CommonTypes:
    FLOATS = [np.float32, np.float16]
    INTS = [np.int32, np.int8, np.uint8]
    BOOL = [np.bool_]


@dataclass
class InputSpec:
    name: str = ""


@dataclass
class ScalarInputSpec(InputSpec):
    default: Any = 0
    choices: Optional[Sequence[Any]] = None


@dataclass
class TensorInputSpec(InputSpec):
    shape_spec: ShapeSpec = None
    dtype_spec: TypeSpec = field(default_factory=lambda: TypeSpec(CommonTypes.FLOATS))
    generator: Optional[Callable[[Tuple[int, ...], Any, np.random.Generator], np.ndarray]] = None

    def make(self, rng: np.random.Generator, shape=None, dtype=None) -> np.ndarray:
        shape = tuple(shape if shape is not None else self.shape_spec.default)
        dtype = np.dtype(dtype if dtype is not None else self.dtype_spec.default)
        if self.generator is not None:
            return self.generator(shape, dtype, rng)
        if dtype.kind == "f":
            return rng.standard_normal(shape).astype(dtype)
        if dtype.kind == "b":
            return rng.random(shape) > 0.5
        return rng.integers(0, 8, shape).astype(dtype)


@dataclass
class KernelSpec:
    function: Callable
    inputs: List[InputSpec]
    is_pure_numpy: bool = True
    description: str = ""

    def default_inputs(self, rng: Optional[np.random.Generator] = None) -> list:
        rng = rng or np.random.default_rng(0)
        return [i.make(rng) if isinstance(i, TensorInputSpec) else i.default for i in self.inputs]
