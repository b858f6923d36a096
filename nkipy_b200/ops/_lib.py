"""ctypes binding of ``libnkipy_b200_kernels.so`` (C ABI in ``csrc/kernels/api.h``).

The library is built in-tree by ``nkipy_b200.ops._build.build()``.  Loading is
lazy; on a machine with a CUDA device a missing library is an error (the ops
never fall back to eager PyTorch on the GPU), on a CPU-only machine the ops use
their PyTorch reference implementations instead.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libnkipy_b200_kernels.so"

_lib = None
_initialised = False

_P = c_void_p
_SIGNATURES = {
    "nkb_init": (c_int, []),
    "nkb_status": (c_int, [c_int]),
    "nkb_set_pdl": (None, [c_int]),
    "nkb_gemm_bf16": (
        c_int,
        [_P, _P, _P, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_int, c_int, c_longlong,
         c_int, c_int, _P, c_int, _P, c_int, c_int, c_int, c_int, _P],
    ),
    "nkb_gemm_bf16_2cta": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, _P, _P, c_int,
                                   c_int, _P]),
    "nkb_gemm_bf16_grouped": (
        c_int,
        [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_int, _P, c_longlong,
         c_float, c_float, c_int, _P, _P, c_int, _P, ctypes.c_uint, _P],
    ),
    "nkb_moe_a2a_dispatch": (c_int, [_P, _P, c_int, c_int, c_int, c_int, c_int, c_int, ctypes.c_uint,
                                     ctypes.POINTER(_P), ctypes.POINTER(_P), ctypes.POINTER(_P), ctypes.POINTER(_P),
                                     ctypes.POINTER(_P), ctypes.POINTER(_P), _P, _P, _P, _P, c_int, c_int, _P, _P,
                                     c_int, _P, _P, _P, _P]),
    "nkb_moe_a2a_combine": (c_int, [_P, _P, c_int, c_int, c_int, c_int, c_int, ctypes.c_uint, ctypes.POINTER(_P),
                                    ctypes.POINTER(_P), ctypes.POINTER(_P), ctypes.POINTER(_P), ctypes.POINTER(_P),
                                    ctypes.POINTER(_P), _P, _P]),
    "nkb_moe_dispatch": (c_int, [_P, c_int, c_int, c_int, c_int, _P, c_int, _P, _P, _P, _P, _P, c_int, _P, _P, c_int,
                                 _P, _P, _P]),
    "nkb_moe_combine": (c_int, [_P, _P, _P, c_int, c_int, c_int, _P, _P]),
    "nkb_gemm_effective_splits": (c_int, [c_int, c_int]),
    "nkb_decode_gemm_splits": (c_int, [c_int, c_int, c_int]),
    "nkb_decode_gemm": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_int,
                                c_int, _P, _P, c_float, c_float, c_int, c_int, _P]),
    "nkb_decode_gemm_push": (c_int, [_P, _P, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, _P, c_int,
                                     ctypes.POINTER(_P), ctypes.POINTER(_P), c_int, c_int, _P, _P, _P, _P]),
    "nkb_decode_gemm_rope": (c_int, [_P, _P, c_int, c_int, c_longlong, c_longlong, c_int, _P, _P, _P, _P, _P, _P,
                                     c_float, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P]),
    "nkb_noalloc_status": (c_int, [c_int]),
    "nkb_gemm_fix_scratch_floats": (c_longlong, [c_int, c_int, c_int, c_int]),
    "nkb_gemm_fix_store": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, _P, _P,
                                   _P, _P, c_int, _P]),
    "nkb_gemm_fix_swiglu": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, _P,
                                    c_float, c_float, _P, _P, c_int, _P]),
    "nkb_gemm_fix_rope": (c_int, [_P, _P, c_int, c_int, c_longlong, c_longlong, c_int, _P, _P, _P, _P, _P, _P, c_float,
                                  _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P, c_int, _P]),
    "nkb_gemm_fix_push": (c_int, [_P, _P, c_int, c_int, c_int, c_longlong, c_longlong, c_int, _P, ctypes.POINTER(_P),
                                  ctypes.POINTER(_P), c_int, c_int, _P, _P, _P, _P, _P, c_int, _P]),
    "nkb_rmsnorm": (c_int, [_P, _P, _P, c_int, c_int, c_float, _P]),
    "nkb_add_rmsnorm": (c_int, [_P, c_int, c_longlong, _P, _P, _P, _P, _P, _P, c_int, c_int, c_float, _P]),
    "nkb_silu_mul": (c_int, [_P, _P, c_int, c_int, c_float, c_float, _P]),
    "nkb_silu_mul_partials": (c_int, [_P, c_int, c_longlong, _P, _P, c_int, c_int, c_float, c_float, _P]),
    "nkb_embedding": (c_int, [_P, _P, _P, c_int, c_int, c_int, _P]),
    "nkb_rope_kv_append": (
        c_int,
        [_P, _P, c_int, c_longlong, _P, _P, _P, _P, _P, _P, c_float, _P, _P, _P, c_int, c_int, c_int, c_int, c_int,
         c_int, _P],
    ),
    "nkb_decode_advance": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "nkb_argmax": (c_int, [_P, c_int, _P, _P, c_int, c_int, c_longlong, _P]),
    "nkb_sample": (c_int, [_P, c_int, _P, c_int, c_int, c_longlong, c_float, c_int, c_float, c_ulonglong,
                           c_ulonglong, _P]),
    "nkb_router_topk": (c_int, [_P, c_int, c_int, c_longlong, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "nkb_paged_attn_decode": (
        c_int,
        [_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, _P,
         c_int, _P],
    ),
    "nkb_paged_attn_decode_fused": (
        c_int,
        [_P, c_int, c_longlong, _P, _P, _P, _P, _P, _P, c_float, c_int, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int,
         c_int, c_int, c_int, c_int, c_float, c_int, _P, c_int, _P],
    ),
    "nkb_paged_attn_decode_scratch_floats": (c_longlong, [c_int, c_int, c_int, c_int, c_int]),
    "nkb_flash_attn_prefill": (
        c_int,
        [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
         c_int, c_int, _P, _P],
    ),
}


class KernelLibraryError(RuntimeError):
    """The native kernel library is missing, failed to load, or a launch failed."""


def available() -> bool:
    return LIB_PATH.exists()


def lib():
    """Load the shared library (once) and declare its signatures."""
    global _lib
    if _lib is not None:
        return _lib
    from . import _build

    # The signatures below are declared from the sources in the tree, so the binary must have been built
    # from exactly those sources: a stale library would be handed shifted arguments.
    if _build.is_stale():
        if os.environ.get("NKIPY_B200_AUTOBUILD", "1") == "1":
            try:
                _build.build()          # takes an inter-process lock; other ranks wait and then find it fresh
            except RuntimeError as e:
                raise KernelLibraryError(f"the kernel library is missing or stale and could not be rebuilt: {e}")
        if _build.is_stale():
            raise KernelLibraryError(
                f"{LIB_PATH} is missing or was built from other sources than csrc/kernels: "
                "run `python -m nkipy_b200.ops._build` (needs nvcc) first"
            )
    handle = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in _SIGNATURES.items():
        try:
            fn = getattr(handle, name)
        except AttributeError:
            continue  # optional entry points are checked at their call site
        fn.restype = res
        fn.argtypes = args
    _lib = handle
    return _lib


def ensure_init():
    """Create the device status word and resolve the TMA encoder (needs a GPU)."""
    global _initialised
    if not _initialised:
        rc = lib().nkb_init()
        if rc != 0:
            raise KernelLibraryError(f"nkb_init failed with code {rc}")
        _initialised = True


def check(rc: int, what: str):
    if rc != 0:
        raise KernelLibraryError(f"{what} failed with code {rc}")


_ERRORS = {
    1: "TMA producer timed out waiting for a free shared-memory stage",
    2: "MMA warp timed out waiting for TMA data",
    3: "MMA warp timed out waiting for the epilogue to free TMEM",
    4: "epilogue timed out waiting for the MMA result",
    5: "a peer or producer flag never arrived",
    6: "bad argument detected on the device",
    7: "MMA warp timed out waiting for the softmax warps",
}


def device_status(reset: bool = True) -> int:
    """Read the device status word (synchronises).  0 means no bounded wait gave up."""
    return int(lib().nkb_status(1 if reset else 0))


def raise_on_device_error():
    code = device_status(reset=True)
    if code:
        raise KernelLibraryError(
            f"device kernel reported status {code & 0xFF} ({_ERRORS.get(code & 0xFF, 'unknown')}) "
            f"from CTA {code >> 8}"
        )
