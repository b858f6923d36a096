"""DeltaNet linear attention as a traced NumPy kernel
(reference: examples/linear_attention/deltanet.py:74-128, torch reference :33-71).

Recurrent delta rule per head, with L2-normalised keys:

    S_t = S_{t-1} + beta_t * (v_t - S_{t-1} k_t) k_t^T          o_t = S_t q_t

The time loop is unrolled while tracing (L is a trace-time constant), so the whole recurrence becomes
one device program of batched [B, H, D, D] x [B, H, D, 1] products and outer products.  The script
runs the kernel on the GPU through `baremetal_jit` when one is present (otherwise in CPU direct mode)
and checks it against a PyTorch implementation of the same recurrence.

    python examples/linear_attention/deltanet.py [--B 1 --H 4 --L 64 --D 32]
"""
import argparse
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))


def deltanet_torch(q, k, v, beta):
    """q, k, v [B, H, L, D], beta [B, H, L] -> o [B, H, L, D]."""
    B, H, L, D = q.shape
    k = k / k.norm(dim=-1, keepdim=True).clamp_min(1e-6)
    S = torch.zeros(B, H, D, D, dtype=q.dtype)
    outs = []
    for t in range(L):
        kt, vt, qt = k[:, :, t], v[:, :, t], q[:, :, t]
        pred = torch.einsum("bhij,bhj->bhi", S, kt)
        S = S + beta[:, :, t, None, None] * torch.einsum("bhi,bhj->bhij", vt - pred, kt)
        outs.append(torch.einsum("bhij,bhj->bhi", S, qt))
    return torch.stack(outs, dim=2)


def deltanet_nkipy(q, k, v, beta):
    """The same recurrence in NumPy operations only (traceable)."""
    B, H, L, D = q.shape
    norm = np.sqrt(np.sum(k * k, axis=-1, keepdims=True))
    k = k / np.maximum(norm, 1e-6)
    S = np.zeros((B, H, D, D), dtype=q.dtype)
    outs = []
    for t in range(L):
        kt = k[:, :, t, :].reshape(B, H, D, 1)
        vt = v[:, :, t, :].reshape(B, H, D, 1)
        qt = q[:, :, t, :].reshape(B, H, D, 1)
        bt = beta[:, :, t].reshape(B, H, 1, 1)
        pred = np.matmul(S, kt)                                        # [B, H, D, 1]
        S = S + bt * np.matmul(vt - pred, kt.reshape(B, H, 1, D))     # outer product
        outs.append(np.matmul(S, qt).reshape(B, H, 1, D))
    return np.concatenate(outs, axis=2)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--B", type=int, default=1)
    ap.add_argument("--H", type=int, default=4)
    ap.add_argument("--L", type=int, default=64)
    ap.add_argument("--D", type=int, default=32)
    ap.add_argument("--cpu", action="store_true", help="CPU direct mode even when a GPU is present")
    args = ap.parse_args()
    rng = np.random.default_rng(0)
    shape = (args.B, args.H, args.L, args.D)
    q, k, v = (rng.standard_normal(shape).astype(np.float32) for _ in range(3))
    beta = (1.0 / (1.0 + np.exp(-rng.standard_normal(shape[:3])))).astype(np.float32)
    want = deltanet_torch(*(torch.from_numpy(a) for a in (q, k, v)), torch.from_numpy(beta)).numpy()
    on_gpu = torch.cuda.is_available() and not args.cpu
    t0 = time.perf_counter()
    if on_gpu:
        from nkipy_b200.runtime import baremetal_jit

        got = baremetal_jit(deltanet_nkipy)(q, k, v, beta)
    else:
        got = deltanet_nkipy(q, k, v, beta)
    dt = time.perf_counter() - t0
    err = float(np.abs(np.asarray(got) - want).max())
    print(f"deltanet B={args.B} H={args.H} L={args.L} D={args.D} on {'gpu' if on_gpu else 'cpu'}: "
          f"{dt:.3f}s (trace + compile + run), max |err| vs torch = {err:.2e}")
    assert err < 1e-3, err
    return 0


if __name__ == "__main__":
    sys.exit(main())
