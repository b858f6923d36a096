"""Spec file: elementwise kernels with free 2-D shapes (the schema is the reference's,
nkipy/src/nkipy/core/specs.py; the import name `nkipy` resolves to this package)."""
import numpy as np
from nkipy.core.specs import CommonTypes, KernelSpec, ScalarInputSpec, ShapeSpec, TensorInputSpec, TypeSpec


def add(a, b):
    return np.add(a, b)


def scaled_residual(x, r, scale):
    return x * scale + r


def hard_sigmoid(x):
    return np.clip(x / 6.0 + 0.5, 0.0, 1.0)


ANY_2D = ShapeSpec(dims=[None, None], default=(32, 32))

kernel_specs = [
    KernelSpec(function=add,
               inputs=[TensorInputSpec(shape_spec=ANY_2D, dtype_spec=CommonTypes.FLOATS, description="lhs"),
                       TensorInputSpec(shape_spec=ANY_2D, dtype_spec=CommonTypes.FLOATS, description="rhs")],
               description="elementwise addition"),
    KernelSpec(function=scaled_residual,
               inputs=[TensorInputSpec(shape_spec=ANY_2D, dtype_spec=CommonTypes.FLOATS),
                       TensorInputSpec(shape_spec=ANY_2D, dtype_spec=CommonTypes.FLOATS),
                       ScalarInputSpec(dtype_spec=TypeSpec(allowed=[float], default=float), default_value=0.5)],
               description="x * scale + residual with a compile-time scale"),
    KernelSpec(function=hard_sigmoid,
               inputs=[TensorInputSpec(shape_spec=ShapeSpec(dims=[(1, 64), (8, 128)], default=(16, 64)),
                                       dtype_spec=CommonTypes.FLOATS)],
               description="clip(x / 6 + 1 / 2, 0, 1)"),
]
