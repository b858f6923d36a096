"""Spec file: attention building blocks -- rotate-halves RoPE, RMSNorm, causal grouped-query attention
(formulated here from the model definitions, batch-free 3-D tensors [tokens, heads, dim])."""
import numpy as np
from nkipy.core.specs import KernelSpec, ShapeSpec, TensorInputSpec, TypeSpec

F32 = TypeSpec(allowed=[np.float32], default=np.float32)


def rmsnorm(x, w):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + 1e-6) * w


def rope(x, cos, sin):
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1)


def gqa_attention(q, k, v):
    t, hq, d = q.shape
    group = hq // k.shape[1]
    kk, vv = np.repeat(k, group, axis=1), np.repeat(v, group, axis=1)
    s = np.matmul(np.transpose(q, (1, 0, 2)), np.transpose(kk, (1, 2, 0))) / np.sqrt(np.float32(d))
    mask = np.triu(np.full((t, t), -1e5, np.float32), k=1)
    s = s + mask
    p = np.exp(s - np.max(s, axis=-1, keepdims=True))
    p = p / np.sum(p, axis=-1, keepdims=True)
    return np.transpose(np.matmul(p, np.transpose(vv, (1, 0, 2))), (1, 0, 2))


def _angles(fn):
    def gen(shape, dtype, rng):
        pos = np.arange(shape[0], dtype=np.float64)[:, None]
        inv = 1.0 / (10000.0 ** (np.arange(shape[1], dtype=np.float64) / shape[1]))
        return fn(pos * inv).astype(dtype)

    return gen


kernel_specs = [
    KernelSpec(function=rmsnorm,
               inputs=[TensorInputSpec(shape_spec=ShapeSpec(dims=[(1, 64), 96], default=(8, 96)), dtype_spec=F32),
                       TensorInputSpec(shape_spec=ShapeSpec(dims=[96], default=(96,)), dtype_spec=F32)],
               description="RMSNorm with fp32 statistics"),
    KernelSpec(function=rope,
               inputs=[TensorInputSpec(shape_spec=ShapeSpec(dims=[12, (1, 6), 32], default=(12, 4, 32)), dtype_spec=F32),
                       TensorInputSpec(shape_spec=ShapeSpec(dims=[12, 16], default=(12, 16)), dtype_spec=F32,
                                       generator=_angles(np.cos)),
                       TensorInputSpec(shape_spec=ShapeSpec(dims=[12, 16], default=(12, 16)), dtype_spec=F32,
                                       generator=_angles(np.sin))],
               description="rotate-halves rotary embedding"),
    KernelSpec(function=gqa_attention,
               inputs=[TensorInputSpec(shape_spec=ShapeSpec(dims=[10, 8, 16], default=(10, 8, 16)), dtype_spec=F32),
                       TensorInputSpec(shape_spec=ShapeSpec(dims=[10, 2, 16], default=(10, 2, 16)), dtype_spec=F32),
                       TensorInputSpec(shape_spec=ShapeSpec(dims=[10, 2, 16], default=(10, 2, 16)), dtype_spec=F32)],
               description="causal grouped-query attention, scores materialised"),
]
