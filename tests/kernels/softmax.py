"""Spec file: row softmax with one and with two outputs."""
import numpy as np
from nkipy.core.specs import CommonTypes, KernelSpec, ShapeSpec, TensorInputSpec


def softmax(x):
    e = np.exp(x - np.max(x, axis=-1, keepdims=True))
    return e / np.sum(e, axis=-1, keepdims=True)


def softmax_and_logsumexp(x):
    m = np.max(x, axis=-1, keepdims=True)
    e = np.exp(x - m)
    s = np.sum(e, axis=-1, keepdims=True)
    return e / s, np.log(s) + m


ROWS = ShapeSpec(dims=[(1, 256), (2, 512)], default=(128, 512))

kernel_specs = [
    KernelSpec(function=softmax, inputs=[TensorInputSpec(shape_spec=ROWS, dtype_spec=CommonTypes.FLOATS)],
               description="softmax along the last axis"),
    KernelSpec(function=softmax_and_logsumexp,
               inputs=[TensorInputSpec(shape_spec=ROWS, dtype_spec=CommonTypes.FLOATS)],
               description="softmax plus its log-sum-exp (two results)"),
]
