"""Spec file: indexing patterns of model code (token gather, head selection, slice assignment, cache update)."""
import numpy as np
from nkipy.core.specs import CommonTypes, KernelSpec, ShapeSpec, TensorInputSpec, TypeSpec

I32 = TypeSpec(allowed=[np.int32], default=np.int32)


def _ids(shape, dtype, rng):
    return rng.integers(0, 50, shape).astype(dtype)


def embedding(table, ids):
    return np.take(table, ids, axis=0)


def select_heads(x):
    # x [tokens, heads, dim]: every other head, last half of the dim, reversed tokens
    return x[::-1, ::2, x.shape[2] // 2:]


def write_slice(cache, new):
    cache[2:2 + new.shape[0], :] = new
    return cache


def last_token_rows(x, lengths):
    return np.take_along_axis(x, (lengths - 1)[:, None, None] + np.zeros((1, 1, x.shape[2]), np.int32), axis=1)[:, 0]


def _lengths(shape, dtype, rng):
    return rng.integers(1, 7, shape).astype(dtype)


kernel_specs = [
    KernelSpec(function=embedding,
               inputs=[TensorInputSpec(shape_spec=ShapeSpec(dims=[50, (4, 64)], default=(50, 32)),
                                       dtype_spec=CommonTypes.FLOATS),
                       TensorInputSpec(shape_spec=ShapeSpec(dims=[(1, 40)], default=(7,)), dtype_spec=I32,
                                       generator=_ids)],
               description="token embedding gather"),
    KernelSpec(function=select_heads,
               inputs=[TensorInputSpec(shape_spec=ShapeSpec(dims=[(1, 16), (2, 8), (2, 32)], default=(5, 4, 16)),
                                       dtype_spec=CommonTypes.FLOATS)],
               description="strided / reversed slicing"),
    KernelSpec(function=write_slice,
               inputs=[TensorInputSpec(shape_spec=ShapeSpec(dims=[16, 8], default=(16, 8)), dtype_spec=CommonTypes.FLOATS),
                       TensorInputSpec(shape_spec=ShapeSpec(dims=[(1, 6), 8], default=(3, 8)),
                                       dtype_spec=CommonTypes.FLOATS)],
               description="slice assignment into a mutated parameter"),
    KernelSpec(function=last_token_rows,
               inputs=[TensorInputSpec(shape_spec=ShapeSpec(dims=[3, 8, (2, 16)], default=(3, 8, 8)),
                                       dtype_spec=CommonTypes.FLOATS),
                       TensorInputSpec(shape_spec=ShapeSpec(dims=[3], default=(3,)), dtype_spec=I32,
                                       generator=_lengths)],
               description="last-token pooling with take_along_axis"),
]
