"""Rotate-halves rotary embedding.  The angle tables depend only on compile-time numbers, so they are plain
NumPy arrays that the trace bakes in as constants (examples/models/qwen3/kernels/rope.py:23-48 in the
reference does the same)."""
import numpy as np


def rope_tables(head_dim: int, max_positions: int, theta: float):
    """cos / sin of shape [max_positions, head_dim / 2], float32."""
    inv_freq = 1.0 / (theta ** (np.arange(0, head_dim, 2, dtype=np.float64) / head_dim))
    ang = np.arange(max_positions, dtype=np.float64)[:, None] * inv_freq[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def rotate_halves(x, cos, sin):
    """x [..., T, heads, D]; cos / sin broadcastable to [..., T, 1, D / 2]."""
    half = x.shape[-1] // 2
    lo, hi = x[..., :half].astype(np.float32), x[..., half:].astype(np.float32)
    out = np.concatenate([lo * cos - hi * sin, hi * cos + lo * sin], axis=-1)
    return out.astype(x.dtype)
