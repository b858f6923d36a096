"""Python side of the persistent decode-layer kernel (csrc/kernels/decode_layer.cu): everything between two
attention calls of a decode step -- o_proj, the sum over ranks or split-K partials with residual and
RMSNorm, gate / up with SwiGLU, down, the second sum and norm, the QKV projection of the next layer with
bias, QK-norm, RoPE and the KV-cache append -- as ONE launch whose CTAs meet at grid-wide barriers.

`decode_layer(**fields)` fills the flat descriptor and launches; `DecodeLayerScratch` owns the fp32 partial
array and the two barrier words of one (device, stream).  The reference compiles a whole layer into one
device program as well (examples/models/qwen3/kernels/transformer_layer.py:17-115).
"""

from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch

from . import _lib

ST_O, ST_RED1, ST_GU, ST_SILU, ST_DOWN, ST_RED2, ST_QKV, ST_ROPE = 1, 2, 4, 8, 16, 32, 64, 128
ST_FFN = ST_GU | ST_DOWN | ST_RED2
ST_ALL = 255

_P, _I, _LL, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_PP = ctypes.POINTER(ctypes.c_void_p)


class _Desc(ctypes.Structure):
    """Field for field the `NkbDecodeLayer` structure of the kernel library."""
    _fields_ = [
        ("mask", _I), ("tokens", _I), ("hidden", _I), ("block_n", _I),
        ("n_ranks", _I), ("rank", _I), ("eps", _F), ("_pad0", _I),
        ("w_o", _P), ("attn", _P), ("ld_wo", _LL), ("ld_attn", _LL), ("k_o", _I), ("splits_o", _I), ("bias_o", _P),
        ("resid_in", _P), ("norm1_w", _P), ("resid_mid", _P), ("normed_mid", _P),
        ("w_gu", _P), ("ld_wgu", _LL), ("inter", _I), ("splits_gu", _I), ("fused_gate", _I), ("_pad1", _I),
        ("bias_gu", _P), ("act_limit", _F), ("act_alpha", _F), ("act", _P),
        ("w_down", _P), ("ld_wdown", _LL), ("splits_down", _I), ("_pad2", _I), ("bias_down", _P),
        ("norm2_w", _P), ("resid_out", _P), ("normed_out", _P),
        ("w_qkv", _P), ("ld_wqkv", _LL), ("splits_qkv", _I), ("nq", _I), ("nkv", _I), ("head_dim", _I),
        ("bias_qkv", _P), ("positions", _P), ("slots", _P), ("cos_sin", _P), ("q_norm_w", _P), ("k_norm_w", _P),
        ("q_out", _P), ("k_cache", _P), ("v_cache", _P), ("max_pos", _I), ("block_size", _I),
        ("scratch", _P), ("scratch_floats", _LL), ("grid_bar", _P),
        ("peer_out_o", _PP), ("peer_flag_o", _PP), ("mc_out_o", _P), ("mc_flag_o", _P),
        ("slabs_o", _P), ("flags_o", _P), ("seen_o", _P), ("done_o", _P),
        ("peer_out_d", _PP), ("peer_flag_d", _PP), ("mc_out_d", _P), ("mc_flag_d", _P),
        ("slabs_d", _P), ("flags_d", _P), ("seen_d", _P), ("done_d", _P),
        ("max_slots", _I), ("_pad3", _I),
        ("red2_x", _P), ("red2_slots", _I), ("_pad4", _I),
        ("timing", _P),
    ]


_checked = False


def _library():
    global _checked
    L = _lib.lib()
    if not _checked:
        L.nkb_decode_layer.restype = _I
        L.nkb_decode_layer.argtypes = [ctypes.POINTER(_Desc), _P]
        L.nkb_decode_layer_desc_size.restype = _I
        L.nkb_decode_layer_desc_size.argtypes = []
        if L.nkb_decode_layer_desc_size() != ctypes.sizeof(_Desc):
            raise _lib.KernelLibraryError(
                f"decode-layer descriptor layout differs: library {L.nkb_decode_layer_desc_size()} bytes, "
                f"binding {ctypes.sizeof(_Desc)} bytes")
        _checked = True
    return L


class DecodeLayerScratch:
    """fp32 split-K partials and the grid-barrier words of the persistent layer kernel for one stream.  The
    barrier words start at zero and return to a consistent state after every launch."""

    MAX_SPLITS = 16

    def __init__(self, device, floats: int):
        self.floats = int(floats)
        self.partials = torch.empty((self.floats,), dtype=torch.float32, device=device)
        self.grid_bar = torch.zeros((4,), dtype=torch.int32, device=device)


_scratch: Dict[Tuple, DecodeLayerScratch] = {}


def scratch_floats(tokens: int, stages) -> int:
    """Floats of partial storage for GEMM stages given as (output width, split factor) pairs."""
    return max([1] + [int(s) * tokens * int(w) for w, s in stages])


def layer_scratch(device, floats: int) -> DecodeLayerScratch:
    """The scratch of the current stream on `device`, grown when a launch needs more."""
    key = (str(device), torch.cuda.current_stream(device).cuda_stream)
    s = _scratch.get(key)
    if s is None or s.floats < floats:
        s = _scratch[key] = DecodeLayerScratch(device, floats)
    return s


def block_n_for(tokens: int) -> int:
    if tokens > 128:
        raise ValueError("the persistent decode-layer kernel takes at most 128 tokens")
    return 32 if tokens <= 32 else (64 if tokens <= 64 else 128)


def pick_layer_splits(rows: int, k: int, sms: int = 148, max_splits: int = 8) -> int:
    """Split-K factor of a GEMM stage that runs on one CTA per SM: the largest factor whose work units
    (row tiles x splits) still fit one wave, as long as every split keeps four 64-wide k-blocks."""
    tiles = (rows + 127) // 128
    kb = max(1, (k + 63) // 64)
    s = max(1, min(sms // max(tiles, 1), kb // 4, max_splits))
    return max(1, s)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def decode_layer(mask: int, tokens: int, hidden: int, eps: float, scratch: DecodeLayerScratch, *,
                 w_o=None, attn=None, splits_o: int = 1, bias_o=None,
                 resid_in=None, norm1_w=None, resid_mid=None, normed_mid=None,
                 w_gu=None, inter: int = 0, splits_gu: int = 1, fused_gate: bool = False, bias_gu=None,
                 act_limit: float = 0.0, act_alpha: float = 1.702, act=None,
                 w_down=None, splits_down: int = 1, bias_down=None,
                 norm2_w=None, resid_out=None, normed_out=None,
                 w_qkv=None, splits_qkv: int = 1, nq: int = 0, nkv: int = 0, head_dim: int = 0, bias_qkv=None,
                 positions=None, slots=None, cos_sin=None, q_norm_w=None, k_norm_w=None,
                 q_out=None, k_cache=None, v_cache=None, tp_buffers=None, red2_x=None, red2_slots: int = 0,
                 timing: Optional[torch.Tensor] = None) -> None:
    """One launch of the persistent layer kernel.  Tensors are bf16 unless the kernel's header says otherwise;
    `mask` selects the stages (ST_*).  ST_RED2 without ST_DOWN sums a block output that other
    kernels produced: `red2_x` [tokens, hidden] on one rank, or `red2_slots` pushed slabs of the second buffer with
    ranks (the residual is `resid_mid`).  timing: int64[80] that receives the device's global
    timer (ns) from CTA 0: [0..15] kernel start and the end of every stage that ran, [16 + 16 g + p] phase p of the
    g-th GEMM stage (entry, set-up done, barrier passed, first operands in shared memory, last MMA issued, first
    accumulator ready, epilogue done, exit, first accumulator chunk in registers, stores of the first tile issued).  tp_buffers: (o, down) buffer descriptions from
    `FusedTP.layer_buffers()` when the row-parallel GEMMs push to the ranks of a tensor-parallel group."""
    from . import _count_launch

    L = _library()
    d = _Desc()
    d.mask, d.tokens, d.hidden, d.block_n = mask, tokens, hidden, block_n_for(tokens)
    d.eps = float(eps)
    if mask & ST_O:
        d.w_o, d.attn = w_o.data_ptr(), attn.data_ptr()
        d.ld_wo, d.ld_attn, d.k_o, d.splits_o = w_o.stride(0), attn.stride(0), w_o.shape[1], splits_o
        d.bias_o = _ptr(bias_o)
    d.resid_in, d.norm1_w, d.resid_mid, d.normed_mid = _ptr(resid_in), _ptr(norm1_w), _ptr(resid_mid), _ptr(normed_mid)
    if mask & ST_GU:
        d.w_gu, d.ld_wgu, d.inter = w_gu.data_ptr(), w_gu.stride(0), inter
        d.splits_gu, d.fused_gate, d.bias_gu = splits_gu, 1 if fused_gate else 0, _ptr(bias_gu)
        d.act_limit, d.act_alpha = float(act_limit), float(act_alpha)
    d.act = _ptr(act)
    if mask & ST_DOWN:
        d.w_down, d.ld_wdown, d.splits_down, d.bias_down = w_down.data_ptr(), w_down.stride(0), splits_down, _ptr(bias_down)
        d.inter = inter
    d.norm2_w, d.resid_out, d.normed_out = _ptr(norm2_w), _ptr(resid_out), _ptr(normed_out)
    d.red2_x, d.red2_slots = _ptr(red2_x), red2_slots
    if timing is not None:
        if timing.dtype != torch.int64 or timing.numel() < 80:
            raise ValueError("timing must be an int64 tensor of 80 elements")
        d.timing = timing.data_ptr()
    if mask & ST_QKV:
        d.w_qkv, d.ld_wqkv, d.splits_qkv = w_qkv.data_ptr(), w_qkv.stride(0), splits_qkv
        d.nq, d.nkv, d.head_dim, d.bias_qkv = nq, nkv, head_dim, _ptr(bias_qkv)
        d.positions, d.slots, d.cos_sin = _ptr(positions), _ptr(slots), _ptr(cos_sin)
        d.q_norm_w, d.k_norm_w = _ptr(q_norm_w), _ptr(k_norm_w)
        d.q_out, d.k_cache, d.v_cache = q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
        d.max_pos = cos_sin.shape[0] if cos_sin is not None else 0
        d.block_size = k_cache.shape[2]
    d.scratch, d.scratch_floats, d.grid_bar = scratch.partials.data_ptr(), scratch.floats, scratch.grid_bar.data_ptr()
    if tp_buffers is not None:
        bo, bd = tp_buffers
        d.n_ranks, d.rank, d.max_slots = bo["n"], bo["rank"], bo["max_slots"]
        for suffix, b in (("o", bo), ("d", bd)):
            setattr(d, "peer_out_" + suffix, ctypes.cast(b["peer_out"], _PP))
            setattr(d, "peer_flag_" + suffix, ctypes.cast(b["peer_flag"], _PP))
            setattr(d, "mc_out_" + suffix, b["mc_out"])
            setattr(d, "mc_flag_" + suffix, b["mc_flag"])
            setattr(d, "slabs_" + suffix, b["slabs"])
            setattr(d, "flags_" + suffix, b["flags"])
            setattr(d, "seen_" + suffix, b["seen"])
            setattr(d, "done_" + suffix, b["done"])
    rc = L.nkb_decode_layer(ctypes.byref(d), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "nkb_decode_layer")
    _count_launch()


def env_splits() -> Optional[Tuple[int, int, int, int]]:
    """``NKIPY_B200_LAYER_SPLITS=o,gu,down,qkv`` overrides the split-K factors of the four GEMM stages
    (0 keeps the heuristic) -- for sweeps."""
    v = os.environ.get("NKIPY_B200_LAYER_SPLITS")
    if not v:
        return None
    parts = [int(x) for x in v.split(",")]
    if len(parts) != 4:
        raise ValueError("NKIPY_B200_LAYER_SPLITS takes four comma-separated integers: o,gu,down,qkv")
    return tuple(parts)
