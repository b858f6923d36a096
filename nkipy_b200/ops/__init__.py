"""Hot-path operators of the model layer.

Every function takes torch tensors.  CUDA tensors are served by the hand-written
sm_100a kernels in ``csrc/kernels`` (tcgen05/TMEM GEMM and prefill attention fed
by TMA, paged decode attention, fused norm / RoPE / cache-append / sampling
kernels) through a C ABI; there is no eager-PyTorch fallback on the GPU — a
missing library raises.  CPU tensors run the plain PyTorch reference of the same
op (fp32 math), which doubles as the oracle in the numerics tests and lets the
models run in CPU-only unit tests.

Weights are kept on the device as ``[out_features, in_features]`` ("NK",
K-major) bf16, the layout both tcgen05 operands want; the safetensors schema of
the reference (``x @ W`` orientation, examples/models/qwen3/tensor_preparation.py:126-248)
is transposed once at load time.
"""

from __future__ import annotations

import os

import math
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import KernelLibraryError, device_status, raise_on_device_error

__all__ = [
    "linear", "decode_linear", "qkv_rope_append", "reduce_partials", "rmsnorm", "add_rmsnorm", "silu_mul", "embedding", "rope_kv_append",
    "argmax", "sample", "decode_advance", "router_topk", "moe_dispatch", "grouped_linear", "moe_combine", "paged_attn_decode", "flash_attn_prefill", "rope_table",
    "KernelLibraryError", "device_status", "raise_on_device_error", "native_available", "launch_count",
    "reset_launch_count",
]

_launches = 0


def launch_count() -> int:
    """Number of native kernel launches issued through this module so far."""
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def _count_launch(n: int = 1) -> None:
    global _launches
    _launches += n


def native_available() -> bool:
    return _lib.available()


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _native(t: torch.Tensor) -> bool:
    if not t.is_cuda:
        return False
    _lib.ensure_init()
    return True


def _check_bf16(*tensors):
    for t in tensors:
        if t is not None and t.dtype != torch.bfloat16:
            raise TypeError(f"expected bfloat16 tensor, got {t.dtype}")


# --------------------------------------------------------------------------- GEMM
_USE_2CTA = os.environ.get("NKIPY_B200_GEMM_2CTA", "1") == "1"


def _pick_block_n(cols: int, gated: bool) -> int:
    cap = 128 if gated else 256
    for bn in (32, 64, 128, 256):
        if cols <= bn and bn <= cap:
            return bn
    return cap


def linear(
    x: torch.Tensor,
    w: torch.Tensor,
    *,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    splits: int = 1,
    gated: bool = False,
    swap: Optional[bool] = None,
    max_ctas: int = 0,
    weights_static: bool = True,
    ctas_per_sm: Optional[int] = None,
) -> torch.Tensor:
    """``y = x @ w.T`` with optional fused epilogue.

    x: [M, K] bf16 (row stride may exceed K), w: [N, K] bf16.
    gated: w is ``[2*I, K]`` holding gate rows then up rows; returns
           ``silu(x @ gate.T) * (x @ up.T)`` of shape [M, I].
    splits > 1: split-K; returns fp32 partial sums ``[S, M, N]`` (S may be smaller
           than requested) for a fused reduction (`add_rmsnorm`, `rope_kv_append`,
           `reduce_partials`).  bias is added to partial 0.
    swap: put the weight on the 128-row MMA side (decode-sized M).  Default: M <= 128.
    ctas_per_sm: 2 halves the shared-memory ring so two CTAs share an SM (default for the
           swapped / decode orientation: lets the next kernel's prefetch overlap this one's tail).
    weights_static: w is not written by the kernels launched just before this one, so its
           tiles may be fetched before the preceding kernel has finished (set False when w is
           itself a fresh activation).
    """
    M, K = x.shape
    N = w.shape[0] // 2 if gated else w.shape[0]
    if w.shape[1] != K:
        raise ValueError(f"shape mismatch: x {tuple(x.shape)} w {tuple(w.shape)}")
    if not _native(x):
        xf, wf = x.float(), w.float()
        if gated:
            g, u = xf @ wf[:N].T, xf @ wf[N:].T
            y = torch.nn.functional.silu(g) * u
        else:
            y = xf @ wf.T
        if bias is not None:
            y = y + bias.float()
        if splits > 1:
            return y.unsqueeze(0)
        if residual is not None:
            y = y + residual.float()
        y = y.to(torch.bfloat16)
        if out is not None:
            out.copy_(y)
            return out
        return y
    global _launches
    _check_bf16(x, w, bias, residual)
    if x.stride(1) != 1 or w.stride(1) != 1:
        raise ValueError("linear needs K-contiguous operands")
    if swap is None:
        swap = M <= 128
    L = _lib.lib()
    if splits > 1:
        eff = L.nkb_gemm_effective_splits(K, splits)
        if out is None:
            out = torch.empty((eff, M, N), dtype=torch.float32, device=x.device)
        elif out.dtype != torch.float32 or out.numel() < eff * M * N:
            raise ValueError("split-K output must be fp32 with room for [S, M, N]")
        out_view = out.view(-1)[: eff * M * N].view(eff, M, N)
        out_fp32, split_stride = 1, M * N
    else:
        eff = 1
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        out_view = out
        out_fp32, split_stride = 0, 0
    ldo = out_view.stride(-2) if out_view.dim() >= 2 else N
    if (not swap and splits <= 1 and M >= 512 and N >= 256 and _USE_2CTA and (ldo & 7) == 0
            and not (gated and (bias is not None or residual is not None))):
        # prefill-sized: CTA pairs on 256 x 256 tiles (csrc/kernels/gemm_2cta.cu)
        rc = L.nkb_gemm_bf16_2cta(x.data_ptr(), w.data_ptr(), out_view.data_ptr(), M, N, K, x.stride(0), w.stride(0),
                                  ldo, _ptr(bias), _ptr(residual), 1 if gated else 0, N if gated else 0, _stream())
        if rc != -5:
            _lib.check(rc, "nkb_gemm_bf16_2cta")
            _launches += 1
            return out_view
    if swap:
        a, b, rows, cols = w, x, N, M
        lda, ldb = w.stride(0), x.stride(0)
        gate_mode = 1 if gated else 0
        block_n = _pick_block_n(cols, gated)
        transpose_out, bias_on_rows = 1, 1
    else:
        a, b, rows, cols = x, w, M, N
        lda, ldb = x.stride(0), w.stride(0)
        gate_mode = 2 if gated else 0
        block_n = 128 if gated else (256 if N >= 256 else _pick_block_n(N, False))
        transpose_out, bias_on_rows = 0, 0
    rc = L.nkb_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out_view.data_ptr(), rows, cols, K, lda, ldb, ldo, transpose_out, out_fp32,
        eff if splits > 1 else 1, split_stride, gate_mode, N if gated else 0, _ptr(bias), bias_on_rows,
        _ptr(residual), block_n, max_ctas, (0 if swap else 1) if weights_static else -1,
        (2 if (swap and not gated) else 1) if ctas_per_sm is None else ctas_per_sm, _stream(),
    )
    _lib.check(rc, "nkb_gemm_bf16")
    _launches += 1
    return out_view


# How the decode projections sum their split-K partials (NKIPY_B200_DECODE_GEMM):
#   legacy  (default) fp32 partials left to the next kernel of the chain (RoPE + append, SwiGLU, residual +
#           RMSNorm), which sums them with the parallelism of a whole grid
#   fixup   inside the persistent GEMM: the CTA that arrives last at a tile's counter sums the partials and
#           applies the epilogue (csrc/kernels/splitk_fix.cuh)
#   cluster thread-block clusters exchanging partials through distributed shared memory
#           (csrc/kernels/gemm_decode.cu)
# Measured on B200 (Llama-3-8B shapes, batch 64): the two fused forms save three launches per layer but lose
# more than that inside the kernel -- the fix-up's one CTA per tile sums with too little memory parallelism,
# cluster launches delay their successors -- so the unfused chain stays the default.
DECODE_GEMM_IMPL = os.environ.get("NKIPY_B200_DECODE_GEMM", "legacy")
# How a decode step runs what lies between two attention calls:
#   persistent  one launch per layer (csrc/kernels/decode_layer.cu): the projections, the sums over ranks or
#               split-K partials, norms, SwiGLU, RoPE and the cache append are stages of one kernel on one CTA
#               per SM that meet at grid-wide barriers
#   chain       one launch per operation (eight or nine per layer)
DECODE_LAYER_IMPL = os.environ.get("NKIPY_B200_DECODE_LAYER", "chain")
_FIX_SCRATCH = {}
_FIX_COUNTERS = 4096


def fix_scratch(device: torch.device, floats: int):
    """(partials fp32, counters int32) scratch of the fix-up GEMMs, one per (device, stream), grown on demand.
    Counters start at zero and every launch leaves them at zero, so consecutive launches share them."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ent = _FIX_SCRATCH.get(key)
    if ent is None or ent[0].numel() < floats:
        part = torch.empty((max(int(floats), 1 << 20),), dtype=torch.float32, device=device)
        ctr = ent[1] if ent is not None else torch.zeros((_FIX_COUNTERS,), dtype=torch.int32, device=device)
        ent = (part, ctr)
        _FIX_SCRATCH[key] = ent
    return ent


def decode_linear(
    x: torch.Tensor,
    w: torch.Tensor,
    *,
    splits: int = 1,
    gated: bool = False,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    ctas_per_sm: int = 2,
    act_limit: float = 0.0,
    act_alpha: float = 1.702,
    impl: Optional[str] = None,
) -> torch.Tensor:
    """``y = x @ w.T`` for a decode-sized batch (at most 128 rows) with the split-K reduction inside the
    kernel, so the result is final bf16.  impl "fixup" (default, see DECODE_GEMM_IMPL): the CTA that
    completes a tile's arrival counter sums the fp32 partials (csrc/kernels/splitk_fix.cuh); "cluster":
    the `splits` CTAs of one 128-feature tile form a cluster and exchange their partial sums through
    distributed shared memory (csrc/kernels/gemm_decode.cu; splits rounded down to a power of two <= 8).
    gated: w holds [gate; up] rows and the result is ``silu(x @ gate.T) * (x @ up.T)`` (act_limit > 0:
    the clamped form ``(up + 1) * gate * sigmoid(act_alpha * gate)``); bias then is [gate bias; up bias].
    splits is rounded down to a power of two (at most 8)."""
    M, K = x.shape
    N = w.shape[0] // 2 if gated else w.shape[0]
    if not _native(x) or M > 128:
        if gated and (act_limit > 0 or bias is not None):
            return silu_mul(linear(x, w, bias=bias), limit=act_limit, alpha=act_alpha, out=out)
        return linear(x, w, bias=bias, residual=residual, out=out, gated=gated)
    global _launches
    _check_bf16(x, w, bias, residual)
    if x.stride(1) != 1 or w.stride(1) != 1:
        raise ValueError("decode_linear needs K-contiguous operands")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    block_n = 32 if M <= 32 else (64 if M <= 64 else 128)
    impl = ("fixup" if DECODE_GEMM_IMPL == "legacy" else DECODE_GEMM_IMPL) if impl is None else impl
    if impl != "cluster" and (not gated or N % 128 == 0) and (2 * N if gated else N) <= 128 * _FIX_COUNTERS:
        L = _lib.lib()
        rows = 2 * N if gated else N
        part, ctr = fix_scratch(x.device, L.nkb_gemm_fix_scratch_floats(rows, M, K, int(splits)))
        if gated:
            rc = L.nkb_gemm_fix_swiglu(w.data_ptr(), x.data_ptr(), out.data_ptr(), N, M, K, w.stride(0), x.stride(0),
                                       out.stride(0), int(splits), _ptr(bias), float(act_limit), float(act_alpha),
                                       part.data_ptr(), ctr.data_ptr(), block_n, _stream())
        else:
            rc = L.nkb_gemm_fix_store(w.data_ptr(), x.data_ptr(), out.data_ptr(), N, M, K, w.stride(0), x.stride(0),
                                      out.stride(0), int(splits), _ptr(bias), _ptr(residual), part.data_ptr(),
                                      ctr.data_ptr(), block_n, _stream())
        _lib.check(rc, "nkb_gemm_fix")
        _launches += 1
        return out
    rc = _lib.lib().nkb_decode_gemm(w.data_ptr(), x.data_ptr(), out.data_ptr(), N, M, K, w.stride(0), x.stride(0),
                                    out.stride(0), int(splits), 1 if gated else 0, N if gated else 0, _ptr(bias),
                                    _ptr(residual), float(act_limit), float(act_alpha), block_n, int(ctas_per_sm),
                                    _stream())
    _lib.check(rc, "nkb_decode_gemm")
    _launches += 1
    return out


def qkv_rope_append(
    x: torch.Tensor,
    w_qkv: torch.Tensor,
    positions: torch.Tensor,
    slots: Optional[torch.Tensor],
    cos_sin: Optional[torch.Tensor],
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    nq: int,
    nkv: int,
    head_dim: int,
    *,
    splits: int = 1,
    bias: Optional[torch.Tensor] = None,
    q_norm_w: Optional[torch.Tensor] = None,
    k_norm_w: Optional[torch.Tensor] = None,
    norm_eps: float = 1e-6,
    q_out: Optional[torch.Tensor] = None,
    impl: Optional[str] = None,
) -> torch.Tensor:
    """The fused QKV projection of a decode step in one launch: ``x @ w_qkv.T`` (+ bias), per-head
    QK-norm, RoPE, K / V written to their cache slots; returns the rotated queries [T, nq * head_dim].
    Equivalent to `linear` followed by `rope_kv_append`."""
    T, K = x.shape
    if not _native(x) or T > 128 or head_dim not in (64, 128):
        qkv = linear(x, w_qkv, swap=True) if _native(x) else linear(x, w_qkv)
        return rope_kv_append(qkv, positions, slots, cos_sin, k_cache, v_cache, nq, nkv, head_dim, bias=bias,
                              q_norm_w=q_norm_w, k_norm_w=k_norm_w, norm_eps=norm_eps, q_out=q_out)
    global _launches
    _check_bf16(x, w_qkv, bias, q_norm_w, k_norm_w)
    if w_qkv.shape[0] != (nq + 2 * nkv) * head_dim:
        raise ValueError("w_qkv rows must be (nq + 2 * nkv) * head_dim")
    if q_out is None:
        q_out = torch.empty((T, nq * head_dim), dtype=torch.bfloat16, device=x.device)
    block_n = 32 if T <= 32 else (64 if T <= 64 else 128)
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    impl = ("fixup" if DECODE_GEMM_IMPL == "legacy" else DECODE_GEMM_IMPL) if impl is None else impl
    if impl != "cluster" and w_qkv.shape[0] <= 128 * _FIX_COUNTERS:
        L = _lib.lib()
        part, ctr = fix_scratch(x.device, L.nkb_gemm_fix_scratch_floats(w_qkv.shape[0], T, K, int(splits)))
        rc = L.nkb_gemm_fix_rope(
            w_qkv.data_ptr(), x.data_ptr(), T, K, w_qkv.stride(0), x.stride(0), int(splits), _ptr(bias),
            _ptr(positions), _ptr(slots), _ptr(cos_sin), _ptr(q_norm_w), _ptr(k_norm_w), float(norm_eps),
            q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), nq, nkv, head_dim, max_pos, k_cache.shape[2],
            part.data_ptr(), ctr.data_ptr(), block_n, _stream())
        _lib.check(rc, "nkb_gemm_fix_rope")
        _launches += 1
        return q_out
    rc = _lib.lib().nkb_decode_gemm_rope(
        w_qkv.data_ptr(), x.data_ptr(), T, K, w_qkv.stride(0), x.stride(0), int(splits), _ptr(bias), _ptr(positions),
        _ptr(slots), _ptr(cos_sin), _ptr(q_norm_w), _ptr(k_norm_w), float(norm_eps), q_out.data_ptr(),
        k_cache.data_ptr(), v_cache.data_ptr(), nq, nkv, head_dim, max_pos, k_cache.shape[2], block_n, _stream())
    _lib.check(rc, "nkb_decode_gemm_rope")
    _launches += 1
    return q_out


def reduce_partials(partials: torch.Tensor, residual: Optional[torch.Tensor] = None,
                    bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sum split-K partials ``[S, M, N]`` (+ bias, + residual) into bf16 ``[M, N]``."""
    S, M, N = partials.shape
    out = torch.empty((M, N), dtype=torch.bfloat16, device=partials.device)
    add_rmsnorm(None, None, residual_in=residual, partials=partials, bias=bias, residual_out=out,
                hidden=N, rows=M)
    return out


# --------------------------------------------------------------------------- norms
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-wise RMSNorm with fp32 statistics; x [..., H] bf16."""
    H = x.shape[-1]
    rows = x.numel() // H
    if out is None:
        out = torch.empty_like(x)
    if not _native(x):
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
        out.copy_(y.to(x.dtype))
        return out
    global _launches
    _check_bf16(x, w)
    rc = _lib.lib().nkb_rmsnorm(x.data_ptr(), w.data_ptr(), out.data_ptr(), rows, H, float(eps), _stream())
    _lib.check(rc, "nkb_rmsnorm")
    _launches += 1
    return out


def add_rmsnorm(
    x: Optional[torch.Tensor],
    w: Optional[torch.Tensor],
    *,
    residual_in: Optional[torch.Tensor] = None,
    partials: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    residual_out: Optional[torch.Tensor] = None,
    normed_out: Optional[torch.Tensor] = None,
    eps: float = 1e-6,
    hidden: Optional[int] = None,
    rows: Optional[int] = None,
) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Fused ``h = sum(partials) + x + bias + residual_in``; ``residual_out = h``;
    ``normed_out = rmsnorm(h) * w``.  Any of x / partials / bias / residual_in may
    be None; w None skips the norm.  Returns (residual_out, normed_out)."""
    ref = x if x is not None else partials
    if hidden is None:
        hidden = ref.shape[-1]
    if rows is None:
        rows = (ref.numel() // hidden) if x is not None else partials.shape[-2]
    dev = ref.device
    if residual_out is None and (residual_in is not None or partials is not None or w is None):
        residual_out = torch.empty((rows, hidden), dtype=torch.bfloat16, device=dev)
    if w is not None and normed_out is None:
        normed_out = torch.empty((rows, hidden), dtype=torch.bfloat16, device=dev)
    if not _native(ref):
        h = torch.zeros((rows, hidden), dtype=torch.float32, device=dev)
        if partials is not None:
            h = h + partials.float().reshape(-1, rows, hidden).sum(0)
        if x is not None:
            h = h + x.float().reshape(rows, hidden)
        if bias is not None:
            h = h + bias.float()
        if residual_in is not None:
            h = h + residual_in.float().reshape(rows, hidden)
        if residual_out is not None:
            residual_out.copy_(h.to(torch.bfloat16).reshape(residual_out.shape))
            h = residual_out.float().reshape(rows, hidden)
        if w is not None:
            y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * w.float()
            normed_out.copy_(y.to(torch.bfloat16).reshape(normed_out.shape))
        return residual_out, normed_out
    global _launches
    _check_bf16(x, w, residual_in, bias)
    splits, stride = 0, 0
    if partials is not None:
        if partials.dtype != torch.float32:
            raise TypeError("partials must be fp32")
        splits = partials.shape[0] if partials.dim() == 3 else 1
        stride = partials.stride(0) if partials.dim() == 3 else 0
    rc = _lib.lib().nkb_add_rmsnorm(
        _ptr(partials), splits, stride, _ptr(x), _ptr(residual_in), _ptr(bias), _ptr(w), _ptr(residual_out),
        _ptr(normed_out), rows, hidden, float(eps), _stream(),
    )
    _lib.check(rc, "nkb_add_rmsnorm")
    _launches += 1
    return residual_out, normed_out


def _silu_mul_partials(parts, out, limit, alpha, bias):
    """SwiGLU gate over fp32 split-K partials [S, T, 2I] (summed on the fly) -> bf16 [T, I]."""
    if parts.dim() == 2:
        parts = parts.unsqueeze(0)
    S, T, two_i = parts.shape
    inter = two_i // 2
    if out is None:
        out = torch.empty((T, inter), dtype=torch.bfloat16, device=parts.device)
    if not _native(parts):
        x = parts.sum(0)
        if bias is not None:
            x = x + bias.float()
        g, u = x[:, :inter], x[:, inter:]
        if limit > 0:
            g = g.clamp(max=limit)
            u = u.clamp(-limit, limit)
            y = (u + 1) * g * torch.sigmoid(alpha * g)
        else:
            y = torch.nn.functional.silu(g) * u
        out.copy_(y.to(torch.bfloat16))
        return out
    global _launches
    rc = _lib.lib().nkb_silu_mul_partials(parts.data_ptr(), S, parts.stride(0), _ptr(bias), out.data_ptr(), T, inter,
                                          float(limit), float(alpha), _stream())
    _lib.check(rc, "nkb_silu_mul_partials")
    _launches += 1
    return out


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, limit: float = 0.0,
             alpha: float = 1.702, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """SwiGLU gate over ``[T, 2I]`` (gate | up) -> ``[T, I]``; limit > 0 selects the
    clamped gpt-oss form ``(up + 1) * gate * sigmoid(alpha * gate)``."""
    if gate_up.dtype == torch.float32:
        return _silu_mul_partials(gate_up, out, limit, alpha, bias)
    T, two_i = gate_up.shape
    inter = two_i // 2
    if out is None:
        out = torch.empty((T, inter), dtype=gate_up.dtype, device=gate_up.device)
    if not _native(gate_up):
        g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
        if limit > 0:
            g = g.clamp(max=limit)
            u = u.clamp(-limit, limit)
            y = (u + 1) * g * torch.sigmoid(alpha * g)
        else:
            y = torch.nn.functional.silu(g) * u
        out.copy_(y.to(gate_up.dtype))
        return out
    global _launches
    _check_bf16(gate_up)
    rc = _lib.lib().nkb_silu_mul(gate_up.data_ptr(), out.data_ptr(), T, inter, float(limit), float(alpha), _stream())
    _lib.check(rc, "nkb_silu_mul")
    _launches += 1
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    n = ids.numel()
    V, H = table.shape
    if out is None:
        out = torch.empty((n, H), dtype=table.dtype, device=table.device)
    if not _native(table):
        out.copy_(table[ids.reshape(-1).long().clamp(0, V - 1)])
        return out
    global _launches
    if ids.dtype != torch.int32:
        ids = ids.to(torch.int32)
    rc = _lib.lib().nkb_embedding(ids.data_ptr(), table.data_ptr(), out.data_ptr(), n, H, V, _stream())
    _lib.check(rc, "nkb_embedding")
    _launches += 1
    return out


# --------------------------------------------------------------------------- rope + kv cache
def rope_table(head_dim: int, max_pos: int, theta: float = 10000.0, inv_freq: Optional[torch.Tensor] = None,
               scaling: float = 1.0, device="cpu") -> torch.Tensor:
    """fp32 table ``[max_pos, head_dim]`` = ``[cos(pos * f) | sin(pos * f)]`` for the
    rotate-halves convention; `inv_freq` (+ `scaling` of cos/sin) carries YaRN."""
    if inv_freq is None:
        inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv_freq.double()[None, :]
    tab = torch.cat([ang.cos(), ang.sin()], dim=-1) * scaling
    return tab.float().to(device)


def rope_kv_append(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    slots: Optional[torch.Tensor],
    cos_sin: Optional[torch.Tensor],
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    nq: int,
    nkv: int,
    head_dim: int,
    *,
    bias: Optional[torch.Tensor] = None,
    q_norm_w: Optional[torch.Tensor] = None,
    k_norm_w: Optional[torch.Tensor] = None,
    norm_eps: float = 1e-6,
    q_out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Split the fused QKV rows, apply optional per-head QK-norm and RoPE, write K/V
    to their cache slots and return the rotated queries ``[T, nq * head_dim]``.

    qkv is bf16 ``[T, W]`` or fp32 split-K partials ``[S, T, W]``.  Cache layout
    ``[num_blocks, nkv, block_size, head_dim]``; slot = block * block_size + offset
    (negative slot = do not store)."""
    partial = qkv.dtype == torch.float32
    T = qkv.shape[-2]
    W = (nq + 2 * nkv) * head_dim
    block_size = k_cache.shape[2]
    if q_out is None:
        q_out = torch.empty((T, nq * head_dim), dtype=torch.bfloat16, device=qkv.device)
    if not _native(qkv):
        x = qkv.float().reshape(-1, T, W).sum(0) if partial else qkv.float()
        if bias is not None:
            x = x + bias.float()
        x = x.reshape(T, nq + 2 * nkv, head_dim)
        q, k, v = x[:, :nq], x[:, nq:nq + nkv], x[:, nq + nkv:]

        def norm(t, w):
            if w is None:
                return t
            y = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + norm_eps) * w.float()
            return y.to(torch.bfloat16).float()

        q, k = norm(q, q_norm_w), norm(k, k_norm_w)
        if cos_sin is not None:
            cs = cos_sin[positions.long().clamp(0, cos_sin.shape[0] - 1)].float()
            c, s = cs[:, None, : head_dim // 2], cs[:, None, head_dim // 2:]

            def rot(t):
                a, b = t[..., : head_dim // 2], t[..., head_dim // 2:]
                return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

            q, k = rot(q), rot(k)
        q_out.copy_(q.reshape(T, nq * head_dim).to(torch.bfloat16))
        if slots is not None:
            sl = slots.long()
            keep = sl >= 0
            blk, off = sl[keep] // block_size, sl[keep] % block_size
            k_cache[blk, :, off] = k[keep].to(k_cache.dtype)
            v_cache[blk, :, off] = v[keep].to(v_cache.dtype)
        return q_out
    global _launches
    L = _lib.lib()
    if partial:
        splits = qkv.shape[0] if qkv.dim() == 3 else 1
        stride = qkv.stride(0) if qkv.dim() == 3 else 0
        bf, pf = None, qkv.data_ptr()
    else:
        _check_bf16(qkv)
        splits, stride, bf, pf = 0, 0, qkv.data_ptr(), None
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    rc = L.nkb_rope_kv_append(
        bf, pf, splits, stride, _ptr(bias), _ptr(positions), _ptr(slots), _ptr(cos_sin), _ptr(q_norm_w),
        _ptr(k_norm_w), float(norm_eps), q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), T, nq, nkv,
        head_dim, max_pos, block_size, _stream(),
    )
    _lib.check(rc, "nkb_rope_kv_append")
    _launches += 1
    return q_out


def decode_advance(context_lens: torch.Tensor, block_table: torch.Tensor, positions: torch.Tensor,
                   slots: torch.Tensor, q_len: int = 1, block_size: int = 32) -> None:
    """Device-side step bookkeeping: positions / cache slots of the q_len new tokens of
    every sequence from its context length and block table, then context_lens += q_len
    (sequences with a negative context length are inactive)."""
    B = context_lens.shape[0]
    if not _native(context_lens):
        ctx = context_lens.long()
        j = torch.arange(q_len)
        pos = ctx[:, None] + j[None, :]
        page = (pos // block_size).clamp(0, block_table.shape[1] - 1)
        blk = block_table.long().gather(1, page)
        sl = blk * block_size + pos % block_size
        active = (ctx >= 0)[:, None].expand_as(pos)
        positions.copy_(torch.where(active, pos, torch.zeros_like(pos)).reshape(-1).to(torch.int32))
        slots.copy_(torch.where(active, sl, torch.full_like(sl, -1)).reshape(-1).to(torch.int32))
        context_lens.copy_(torch.where(ctx >= 0, ctx + q_len, ctx).to(torch.int32))
        return
    global _launches
    rc = _lib.lib().nkb_decode_advance(context_lens.data_ptr(), block_table.data_ptr(), positions.data_ptr(),
                                       slots.data_ptr(), B, q_len, block_table.stride(0), block_size, _stream())
    _lib.check(rc, "nkb_decode_advance")
    _launches += 2


# --------------------------------------------------------------------------- sampling / routing
def argmax(logits: torch.Tensor, out_ids: Optional[torch.Tensor] = None,
           out_vals: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-wise argmax (first occurrence) of bf16/fp32 ``[B, V]`` logits -> int32 ids."""
    B, V = logits.shape
    if out_ids is None:
        out_ids = torch.empty((B,), dtype=torch.int32, device=logits.device)
    if not _native(logits):
        vals, ids = logits.float().max(dim=-1)
        out_ids.copy_(ids.to(torch.int32))
        if out_vals is not None:
            out_vals.copy_(vals)
        return out_ids
    global _launches
    is_fp32 = 1 if logits.dtype == torch.float32 else 0
    rc = _lib.lib().nkb_argmax(logits.data_ptr(), is_fp32, out_ids.data_ptr(), _ptr(out_vals), B, V,
                               logits.stride(0), _stream())
    _lib.check(rc, "nkb_argmax")
    _launches += 1
    return out_ids


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0,
           step: int = 0, out_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Temperature / top-k / top-p sampling.  Candidates are limited to the 1024 most
    likely tokens of each row (the nucleus is taken inside that set)."""
    B, V = logits.shape
    if out_ids is None:
        out_ids = torch.empty((B,), dtype=torch.int32, device=logits.device)
    if not _native(logits):
        g = torch.Generator(device="cpu").manual_seed(seed * 1000003 + step)
        k = min(top_k if 0 < top_k < 1024 else 1024, V)
        vals, idx = logits.float().topk(k, dim=-1)
        probs = torch.softmax(vals / max(temperature, 1e-6), dim=-1)
        if 0 < top_p < 1:
            c = probs.cumsum(-1)
            keep = (c - probs) < top_p
            probs = probs * keep
        pick = torch.multinomial(probs / probs.sum(-1, keepdim=True), 1, generator=g)
        out_ids.copy_(idx.gather(-1, pick).squeeze(-1).to(torch.int32))
        return out_ids
    global _launches
    is_fp32 = 1 if logits.dtype == torch.float32 else 0
    rc = _lib.lib().nkb_sample(logits.data_ptr(), is_fp32, out_ids.data_ptr(), B, V, logits.stride(0),
                               float(temperature), int(top_k), float(top_p), int(seed), int(step), _stream())
    _lib.check(rc, "nkb_sample")
    _launches += 1
    return out_ids


def router_topk(logits: torch.Tensor, top_k: int, mode: str = "softmax_topk",
                bias: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """MoE routing.  mode "softmax_topk": softmax over all experts, top-k, renormalise
    (Qwen3); "topk_softmax": top-k raw logits, softmax over them (gpt-oss).  logits are bf16 /
    fp32 ``[T, E]`` or fp32 split-K partials ``[S, T, E]`` (summed here); bias [E] is added first.
    Returns (weights fp32 [T, k], experts int32 [T, k])."""
    partial = logits.dim() == 3
    T, E = logits.shape[-2], logits.shape[-1]
    if not _native(logits):
        lf = logits.float().sum(0) if partial else logits.float()
        if bias is not None:
            lf = lf + bias.float()
        if mode == "softmax_topk":
            p = torch.softmax(lf, dim=-1)
            w, e = p.topk(top_k, dim=-1)
            w = w / w.sum(-1, keepdim=True)
        else:
            v, e = lf.topk(top_k, dim=-1)
            w = torch.softmax(v, dim=-1)
        return w, e.to(torch.int32)
    global _launches
    w = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    e = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    is_fp32 = 1 if logits.dtype == torch.float32 else 0
    if not logits.is_contiguous():
        logits = logits.contiguous()
    splits = logits.shape[0] if partial else 1
    rc = _lib.lib().nkb_router_topk(logits.data_ptr(), is_fp32, splits, logits.stride(0) if partial else 0, _ptr(bias),
                                    w.data_ptr(), e.data_ptr(), T, E, top_k, 0 if mode == "softmax_topk" else 1,
                                    _stream())
    _lib.check(rc, "nkb_router_topk")
    _launches += 1
    return w, e


# --------------------------------------------------------------------------- attention
def _gather_kv(cache: torch.Tensor, table_row: torch.Tensor, ctx: int) -> torch.Tensor:
    """[ctx, nkv, D] view of one sequence's cached K or V (reference path)."""
    bs = cache.shape[2]
    nblk = (ctx + bs - 1) // bs
    blocks = cache[table_row[:nblk].long()]  # [nblk, nkv, bs, D]
    return blocks.permute(0, 2, 1, 3).reshape(nblk * bs, cache.shape[1], cache.shape[3])[:ctx]


def _ref_attention(q, k, v, scale, q_pos0, causal, window, sinks):
    """q [Lq, nq, D], k/v [Lk, nkv, D] fp32 -> [Lq, nq, D]; query i sits at kv position q_pos0 + i."""
    Lq, nq, D = q.shape
    Lk, nkv, _ = k.shape
    group = nq // nkv
    kk = k.repeat_interleave(group, dim=1)
    vv = v.repeat_interleave(group, dim=1)
    s = torch.einsum("qhd,khd->hqk", q, kk) * scale
    qpos = q_pos0 + torch.arange(Lq, device=q.device)[:, None]
    kpos = torch.arange(Lk, device=q.device)[None, :]
    mask = torch.ones((Lq, Lk), dtype=torch.bool, device=q.device)
    if causal:
        mask &= kpos <= qpos
    if window and window > 0:
        mask &= kpos > qpos - window
    s = s.masked_fill(~mask[None], float("-inf"))
    if sinks is not None:
        s = torch.cat([s, sinks.float()[:, None, None].expand(nq, Lq, 1)], dim=-1)
        p = torch.softmax(s, dim=-1)[..., :-1]
    else:
        p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.einsum("hqk,khd->qhd", p, vv)


def pick_kv_splits(ctas: int, max_pages: int, sms: int = 148) -> int:
    """KV split count for decode attention.  Every warp of the kernel streams its own pages, an SM holds four
    warps, and the kernel picks 4 / 2 / 1 warps per CTA so that the grid stays within one wave.  Splitting
    only pays while the unsplit grid leaves SMs without a CTA: then split until about one four-warp CTA sits
    on every SM, keeping at least two pages per warp."""
    if ctas >= sms:
        return 1
    s = min(sms // ctas, max(max_pages // 8, 1), 16)
    return max(s, 1)


_DECODE_SCRATCH = {}


def _decode_scratch(device: torch.device, floats: int) -> torch.Tensor:
    """Split-KV scratch of the decode attention, one per (device, stream): it starts with the arrival
    counters of the split merge, which must be zero before the first call (the merging CTA resets them),
    so the buffer is zero-filled once and then reused by every call on that stream."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _DECODE_SCRATCH.get(key)
    if buf is None or buf.numel() < floats:
        buf = torch.zeros((int(floats),), dtype=torch.float32, device=device)
        _DECODE_SCRATCH[key] = buf
    return buf


def paged_attn_decode(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    context_lens: torch.Tensor,
    scale: float,
    *,
    q_len: int = 1,
    window: int = 0,
    sinks: Optional[torch.Tensor] = None,
    num_splits: int = 0,
    scratch: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Decode attention over the paged cache.  q ``[B * q_len, nq * D]`` (the q_len
    newest tokens of each sequence, already appended to the cache);
    context_lens counts them.  Causal among the new tokens."""
    nkv, bs, D = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    B = block_table.shape[0]
    nq = q.shape[-1] // D
    if out is None:
        out = torch.empty_like(q)
    if not _native(q):
        qf = q.float().reshape(B, q_len, nq, D)
        res = torch.empty_like(qf)
        for b in range(B):
            ctx = int(context_lens[b])
            k = _gather_kv(k_cache, block_table[b], ctx).float()
            v = _gather_kv(v_cache, block_table[b], ctx).float()
            res[b] = _ref_attention(qf[b], k, v, scale, ctx - q_len, True, window, sinks)
        out.copy_(res.reshape(out.shape).to(out.dtype))
        return out
    global _launches
    _check_bf16(q, k_cache, v_cache)
    if q_len * (nq // nkv) > 16:
        # more query rows per kv head than the decode kernel's 16-row fragment: the blockwise prefill
        # kernel handles any window (query i of a sequence sits at position context_len - q_len + i)
        q_start = torch.arange(B, device=q.device, dtype=torch.int32) * q_len
        q_lens = torch.full((B,), q_len, device=q.device, dtype=torch.int32)
        return flash_attn_prefill(q, k_cache, v_cache, block_table, q_start, q_lens, context_lens, scale,
                                  max_q_len=q_len, causal=True, window=window, sinks=sinks, out=out)
    L = _lib.lib()
    if num_splits <= 0:
        num_splits = pick_kv_splits(B * nkv, block_table.shape[1])
    if num_splits > 1:
        need = L.nkb_paged_attn_decode_scratch_floats(B, q_len, nq, D, num_splits)
        if scratch is None or scratch.numel() < need:
            scratch = _decode_scratch(q.device, need)
    rc = L.nkb_paged_attn_decode(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(), context_lens.data_ptr(),
        out.data_ptr(), _ptr(scratch), B, q_len, nq, nkv, D, bs, k_cache.shape[0], block_table.stride(0),
        float(scale), int(window), _ptr(sinks), num_splits, _stream(),
    )
    _lib.check(rc, "nkb_paged_attn_decode")
    _launches += 1
    return out


# Decode attention reads the fused QKV projection's split-K partials itself (bias, QK-norm, RoPE and the cache
# append included) instead of running after a separate RoPE + append launch.  "1" = always, "0" = never, "auto"
# (default) = on one rank only: the fusion is time-neutral inside the CUDA graph and its multi-rank runs have not
# been re-validated.
FUSED_ROPE_ATTN = os.environ.get("NKIPY_B200_FUSED_ROPE_ATTN", "auto")


def fused_rope_attn_enabled(world_size: int) -> bool:
    if FUSED_ROPE_ATTN == "auto":
        return world_size == 1
    return FUSED_ROPE_ATTN != "0"


def rope_attn_decode(
    qkv_partials: torch.Tensor,
    positions: torch.Tensor,
    slots: torch.Tensor,
    cos_sin: Optional[torch.Tensor],
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    context_lens: torch.Tensor,
    scale: float,
    nq: int,
    nkv: int,
    *,
    bias: Optional[torch.Tensor] = None,
    q_norm_w: Optional[torch.Tensor] = None,
    k_norm_w: Optional[torch.Tensor] = None,
    norm_eps: float = 1e-6,
    window: int = 0,
    sinks: Optional[torch.Tensor] = None,
    num_splits: int = 0,
    scratch: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One new token per sequence: ``rope_kv_append`` followed by ``paged_attn_decode`` as one launch.

    qkv_partials is the fp32 split-K output ``[S, B, (nq + 2 nkv) * D]`` of the fused QKV projection.  The kernel
    sums it, adds the bias, applies QK-norm and RoPE, stores the new key and value at ``slots`` and attends over the
    cache pages plus the new token.  Returns ``[B, nq * D]`` bf16."""
    D = k_cache.shape[3]
    B = block_table.shape[0]
    if out is None:
        out = torch.empty((B, nq * D), dtype=torch.bfloat16, device=qkv_partials.device)
    if not _native(qkv_partials):
        q = rope_kv_append(qkv_partials, positions, slots, cos_sin, k_cache, v_cache, nq, nkv, D, bias=bias,
                           q_norm_w=q_norm_w, k_norm_w=k_norm_w, norm_eps=norm_eps)
        return paged_attn_decode(q, k_cache, v_cache, block_table, context_lens, scale, window=window, sinks=sinks,
                                 out=out)
    global _launches
    _check_bf16(k_cache, v_cache)
    if qkv_partials.dtype != torch.float32 or qkv_partials.shape[-2] != B or nq // nkv > 16:
        raise ValueError("rope_attn_decode wants fp32 partials [S, B, W], one token per sequence, group <= 16")
    L = _lib.lib()
    splits = qkv_partials.shape[0] if qkv_partials.dim() == 3 else 1
    stride = qkv_partials.stride(0) if qkv_partials.dim() == 3 else 0
    bs = k_cache.shape[2]
    if num_splits <= 0:
        num_splits = pick_kv_splits(B * nkv, block_table.shape[1])
    if num_splits > 1:
        need = L.nkb_paged_attn_decode_scratch_floats(B, 1, nq, D, num_splits)
        if scratch is None or scratch.numel() < need:
            scratch = _decode_scratch(qkv_partials.device, need)
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    rc = L.nkb_paged_attn_decode_fused(
        qkv_partials.data_ptr(), splits, stride, _ptr(bias), _ptr(positions), _ptr(slots), _ptr(cos_sin),
        _ptr(q_norm_w), _ptr(k_norm_w), float(norm_eps), max_pos, k_cache.data_ptr(), v_cache.data_ptr(),
        block_table.data_ptr(), context_lens.data_ptr(), out.data_ptr(), _ptr(scratch), B, nq, nkv, D, bs,
        k_cache.shape[0], block_table.stride(0), float(scale), int(window), _ptr(sinks), num_splits, _stream(),
    )
    _lib.check(rc, "nkb_paged_attn_decode_fused")
    _launches += 1
    return out


def flash_attn_prefill(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    q_start: torch.Tensor,
    q_lens: torch.Tensor,
    context_lens: torch.Tensor,
    scale: float,
    *,
    max_q_len: int,
    causal: bool = True,
    window: int = 0,
    sinks: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Blockwise prefill attention.  q ``[total_q, nq * D]`` packs the new tokens of
    all sequences (sequence b owns rows q_start[b] .. q_start[b] + q_lens[b]); K/V
    of the whole context (cached prefix + new tokens) are read from the paged
    cache.  Query i of a sequence sits at position context_len - q_len + i."""
    nkv, bs, D = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    B = block_table.shape[0]
    total_q = q.shape[0]
    nq = q.shape[-1] // D
    if out is None:
        out = torch.empty_like(q)
    if not _native(q):
        qf = q.float().reshape(total_q, nq, D)
        res = torch.zeros_like(qf)
        for b in range(B):
            ctx, ql, qs = int(context_lens[b]), int(q_lens[b]), int(q_start[b])
            if ql == 0:
                continue
            k = _gather_kv(k_cache, block_table[b], ctx).float()
            v = _gather_kv(v_cache, block_table[b], ctx).float()
            res[qs:qs + ql] = _ref_attention(qf[qs:qs + ql], k, v, scale, ctx - ql, causal, window, sinks)
        out.copy_(res.reshape(out.shape).to(out.dtype))
        return out
    global _launches
    _check_bf16(q, k_cache, v_cache)
    rc = _lib.lib().nkb_flash_attn_prefill(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(), q_start.data_ptr(),
        q_lens.data_ptr(), context_lens.data_ptr(), out.data_ptr(), B, total_q, int(max_q_len), nq, nkv, D, bs,
        k_cache.shape[0], block_table.stride(0), float(scale), 1 if causal else 0, int(window), _ptr(sinks),
        _stream(),
    )
    _lib.check(rc, "nkb_flash_attn_prefill")
    _launches += 1
    return out


# --------------------------------------------------------------------------- mixture of experts
class MoEPlan:
    """Result of `moe_dispatch`: expert-sorted rows plus the device-side schedules of the grouped GEMMs."""
    __slots__ = ("x_sorted", "offsets", "pair_pos", "tiles", "max_rows")

    def __init__(self, x_sorted, offsets, pair_pos, tiles, max_rows):
        self.x_sorted, self.offsets, self.pair_pos, self.tiles, self.max_rows = x_sorted, offsets, pair_pos, tiles, max_rows

    def __iter__(self):          # (x_sorted, offsets, pair_pos) unpacking
        return iter((self.x_sorted, self.offsets, self.pair_pos))


def moe_tile_widths(tokens: int):
    """(gated GEMM tile width, down GEMM tile width) in tokens for a batch of `tokens`."""
    if tokens <= 512:
        return 32, 32
    return 64, 128


def moe_dispatch(x: torch.Tensor, experts: torch.Tensor, expert_lo: int, num_local: int) -> MoEPlan:
    """Sort the (token, expert) pairs routed to local experts [expert_lo, expert_lo + num_local) by
    expert and gather their token rows.  x [T, H] bf16, experts [T, k] int32 (global ids).
    Returns a `MoEPlan` (unpacks to x_sorted [T * k, H], offsets int32 [num_local + 1], pair_pos int32
    [T * k]); rows past offsets[-1] of x_sorted are unspecified, pair_pos is -1 for pairs of other
    ranks' experts."""
    T, H = x.shape
    k = experts.shape[1]
    pairs = T * k
    dev = x.device
    if not _native(x):
        flat = experts.reshape(-1).long() - expert_lo
        local = (flat >= 0) & (flat < num_local)
        order = torch.argsort(torch.where(local, flat, torch.full_like(flat, num_local)), stable=True)
        n_local = int(local.sum())
        pair_pos = torch.full((pairs,), -1, dtype=torch.int32)
        pair_pos[order[:n_local]] = torch.arange(n_local, dtype=torch.int32)
        counts = torch.bincount(flat[local], minlength=num_local)
        offsets = torch.zeros((num_local + 1,), dtype=torch.int32)
        offsets[1:] = counts.cumsum(0).to(torch.int32)
        x_sorted = torch.zeros((pairs, H), dtype=x.dtype)
        x_sorted[:n_local] = x[(order[:n_local] // k)]
        return MoEPlan(x_sorted, offsets, pair_pos, None, T)
    global _launches
    bn_a, bn_b = moe_tile_widths(T)
    cap_a, cap_b = num_local + pairs // bn_a + 1, num_local + pairs // bn_b + 1
    x_sorted = torch.empty((pairs, H), dtype=x.dtype, device=dev)
    work = torch.empty((3 * num_local + 1 + pairs + 2 * cap_a + 2 * cap_b + 2,), dtype=torch.int32, device=dev)
    o = 0
    counts = work[o:o + num_local]; o += num_local
    offsets = work[o:o + num_local + 1]; o += num_local + 1
    cursors = work[o:o + num_local]; o += num_local
    pair_pos = work[o:o + pairs]; o += pairs
    tiles_a = work[o:o + 2 * cap_a]; o += 2 * cap_a
    tiles_b = work[o:o + 2 * cap_b]; o += 2 * cap_b
    ntiles = work[o:o + 2]
    if experts.dtype != torch.int32:
        experts = experts.to(torch.int32)
    rc = _lib.lib().nkb_moe_dispatch(experts.data_ptr(), T, k, int(expert_lo), int(num_local), x.data_ptr(), H,
                                     x_sorted.data_ptr(), counts.data_ptr(), offsets.data_ptr(), cursors.data_ptr(),
                                     pair_pos.data_ptr(), bn_a, tiles_a.data_ptr(), ntiles.data_ptr(), bn_b,
                                     tiles_b.data_ptr(), ntiles.data_ptr() + 4, _stream())
    _lib.check(rc, "nkb_moe_dispatch")
    _launches += 2 if pairs <= 8192 else 5
    tiles = {bn_a: (tiles_a, ntiles[0:1], cap_a)}
    tiles.setdefault(bn_b, (tiles_b, ntiles[1:2], cap_b))
    return MoEPlan(x_sorted, offsets, pair_pos, tiles, T)


def grouped_linear(x_sorted: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, *, max_rows_per_group: int,
                   gated: bool = False, bias: Optional[torch.Tensor] = None, act_limit: float = 0.0,
                   act_alpha: float = 1.702, tiles=None, out: Optional[torch.Tensor] = None,
                   arrive: Optional[int] = None, arrive_target: int = 0) -> torch.Tensor:
    """Per-group ``y[r] = x_sorted[r] @ w[g(r)].T`` for rows sorted by group (group g owns rows
    offsets[g] .. offsets[g + 1]).  w [G, N, K] bf16 (gated: [G, 2 * I, K], gate rows then up
    rows, output ``act(gate) * up`` of width I).  bias [G, N] is added before the activation."""
    R, K = x_sorted.shape
    G = w.shape[0]
    N = w.shape[1] // 2 if gated else w.shape[1]
    if not _native(x_sorted):
        out = torch.zeros((R, N), dtype=torch.bfloat16)
        off = offsets.tolist()
        for g in range(G):
            a, b = off[g], off[g + 1]
            if b <= a:
                continue
            y = x_sorted[a:b].float() @ w[g].float().T
            if bias is not None:
                y = y + bias[g].float()
            if gated:
                gg, uu = y[:, :N], y[:, N:]
                if act_limit > 0:
                    gg = gg.clamp(max=act_limit)
                    uu = uu.clamp(-act_limit, act_limit)
                    y = (uu + 1) * gg * torch.sigmoid(act_alpha * gg)
                else:
                    y = torch.nn.functional.silu(gg) * uu
            out[a:b] = y.to(torch.bfloat16)
        return out
    global _launches
    _check_bf16(x_sorted, w, bias)
    if out is None:
        out = torch.empty((R, N), dtype=torch.bfloat16, device=x_sorted.device)
    tl = tc = None
    max_tiles = 0
    if tiles is not None:
        bn_a, bn_b = moe_tile_widths(max_rows_per_group)
        block_n = bn_a if gated else bn_b
        tl_t, tc_t, max_tiles = tiles[block_n]
        tl, tc = tl_t.data_ptr(), tc_t.data_ptr()
    else:
        block_n = 32 if max_rows_per_group <= 32 else 64
        if not gated and max_rows_per_group > 64:
            block_n = 128
    rc = _lib.lib().nkb_gemm_bf16_grouped(
        w.data_ptr(), x_sorted.data_ptr(), out.data_ptr(), offsets.data_ptr(), G, N, K, R, int(max_rows_per_group),
        x_sorted.stride(0), N, 1 if gated else 0, N if gated else 0, _ptr(bias),
        bias.stride(0) if bias is not None else 0, float(act_limit), float(act_alpha), block_n, tl, tc,
        int(max_tiles), arrive, int(arrive_target), _stream())
    _lib.check(rc, "nkb_gemm_bf16_grouped")
    _launches += 1
    return out


def moe_combine(y_sorted: torch.Tensor, pair_pos: torch.Tensor, weights: torch.Tensor, tokens: int) -> torch.Tensor:
    """``out[t] = sum_j weights[t, j] * y_sorted[pair_pos[t * k + j]]`` over local pairs -> bf16 [T, H]."""
    k = weights.shape[1]
    H = y_sorted.shape[1]
    if not _native(y_sorted):
        pos = pair_pos.reshape(tokens, k).long()
        valid = pos >= 0
        rows = y_sorted[pos.clamp(min=0)].float() * (weights.float() * valid)[..., None]
        return rows.sum(1).to(torch.bfloat16)
    global _launches
    out = torch.empty((tokens, H), dtype=torch.bfloat16, device=y_sorted.device)
    if weights.dtype != torch.float32:
        weights = weights.float()
    rc = _lib.lib().nkb_moe_combine(y_sorted.data_ptr(), pair_pos.data_ptr(), weights.data_ptr(), tokens, k, H,
                                    out.data_ptr(), _stream())
    _lib.check(rc, "nkb_moe_combine")
    _launches += 1
    return out
