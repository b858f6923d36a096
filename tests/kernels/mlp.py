"""Spec file: feed-forward blocks (tanh-GELU MLP and SwiGLU), matrices stored in `x @ W` orientation."""
import numpy as np
from nkipy.core.specs import KernelSpec, ShapeSpec, TensorInputSpec, TypeSpec

F32 = TypeSpec(allowed=[np.float32], default=np.float32)


def _small(shape, dtype, rng):
    return (rng.standard_normal(shape) * 0.05).astype(dtype)


def gelu_mlp(x, w1, w2):
    h = x @ w1
    h = 0.5 * h * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (h + 0.044715 * h ** 3)))
    return h @ w2


def swiglu(x, gate_up, down):
    inter = down.shape[0]
    gu = x @ gate_up
    g, u = gu[:, :inter], gu[:, inter:]
    return (g / (1.0 + np.exp(-g)) * u) @ down


kernel_specs = [
    KernelSpec(function=gelu_mlp,
               inputs=[TensorInputSpec(shape_spec=ShapeSpec(dims=[(1, 128), 256], default=(64, 256)), dtype_spec=F32),
                       TensorInputSpec(shape_spec=ShapeSpec(dims=[256, 1024], default=(256, 1024)), dtype_spec=F32,
                                       generator=_small),
                       TensorInputSpec(shape_spec=ShapeSpec(dims=[1024, 256], default=(1024, 256)), dtype_spec=F32,
                                       generator=_small)],
               description="y = gelu(x W1) W2"),
    KernelSpec(function=swiglu,
               inputs=[TensorInputSpec(shape_spec=ShapeSpec(dims=[(1, 64), 128], default=(16, 128)), dtype_spec=F32),
                       TensorInputSpec(shape_spec=ShapeSpec(dims=[128, 512], default=(128, 512)), dtype_spec=F32,
                                       generator=_small),
                       TensorInputSpec(shape_spec=ShapeSpec(dims=[256, 128], default=(256, 128)), dtype_spec=F32,
                                       generator=_small)],
               description="SwiGLU feed-forward with fused gate|up weights"),
]
