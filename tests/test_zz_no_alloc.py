"""Allocation-free decode attention: the exported C symbol against the regular entry point.

Some callers of this library must not allocate device memory while they run (a
serving loop with a frozen memory budget, code living inside another framework's
arena).  `nkb_paged_attn_decode_noalloc` serves them by keeping the split-KV
scratch in a fixed array inside the library.  This file is collected last on
purpose, so a run that stops at the first failure has already run everything else.
"""
import ctypes
import math

import pytest
import torch

from nkipy_b200 import ops
from nkipy_b200.ops import _lib

pytestmark = pytest.mark.gpu

_P = ctypes.c_void_p
_I = ctypes.c_int


def _symbol():
    fn = _lib.lib().nkb_paged_attn_decode_noalloc
    fn.restype = _I
    fn.argtypes = [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, ctypes.c_float, _I, _P, _I, _P]
    return fn


def _case(B, ctx_lens, nq, nkv, D, seed):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed)
    max_blocks = (max(ctx_lens) + 31) // 32
    nb = B * max_blocks + 3
    kc = (torch.randn(nb, nkv, 32, D, device=dev, generator=g)).to(torch.bfloat16)
    vc = (torch.randn(nb, nkv, 32, D, device=dev, generator=g)).to(torch.bfloat16)
    table = torch.randperm(nb, device=dev)[: B * max_blocks].reshape(B, max_blocks).to(torch.int32)
    lens = torch.tensor(ctx_lens, device=dev, dtype=torch.int32)
    q = torch.randn(B, nq * D, device=dev, generator=g).to(torch.bfloat16)
    return q, kc, vc, table, lens


def _run_both(fn, B, ctx_lens, nq, nkv, D, splits, seed):
    q, kc, vc, table, lens = _case(B, ctx_lens, nq, nkv, D, seed)
    scale = 1.0 / math.sqrt(D)
    expect = ops.paged_attn_decode(q, kc, vc, table, lens, scale, num_splits=splits)
    out = torch.empty_like(q)
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), lens.data_ptr(), out.data_ptr(), B, 1, nq,
            nkv, D, 32, kc.shape[0], table.stride(0), scale, 0, None, splits,
            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    err = ((out.float() - expect.float()).norm() / expect.float().norm()).item()
    assert err < 2e-2, err
    return out


def test_noalloc_matches_regular_entry_point_twice():
    fn = _symbol()
    # two calls in a row share the built-in scratch array; the second is a different problem
    _run_both(fn, 6, [700, 33, 1025, 64, 300, 512], 8, 2, 128, 4, seed=1)
    _run_both(fn, 3, [260, 900, 31], 8, 8, 64, 2, seed=2)
    _run_both(fn, 6, [700, 33, 1025, 64, 300, 512], 8, 2, 128, 1, seed=3)


def test_noalloc_rejects_oversized_problem():
    fn = _symbol()
    q, kc, vc, table, lens = _case(2, [64, 64], 8, 8, 128, 4)
    out = torch.empty_like(q)
    # batch 4096 x 8 kv heads x 16 splits x 2080 floats is far beyond the 4 Mi-float array: nothing may launch
    rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), lens.data_ptr(), out.data_ptr(), 4096, 1, 8,
            8, 128, 32, kc.shape[0], table.stride(0), 0.1, 0, None, 16, torch.cuda.current_stream().cuda_stream)
    assert rc == -10
