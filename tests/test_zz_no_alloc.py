"""Allocation-free decode attention: the exported C symbol against the regular entry point.

Some callers of this library must not allocate device memory while they run (a
serving loop with a frozen memory budget, code living inside another framework's
arena).  `nkb_paged_attn_decode_noalloc` serves them by keeping the split-KV
scratch in a fixed array inside the library.  This file is collected last on
purpose, so a run that stops at the first failure has already run everything else.
"""
import ctypes
import math
import os
import subprocess
import sys
import textwrap

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
    # a bounded wait that gave up inside this entry point reports into its own status word
    assert _lib.lib().nkb_noalloc_status(1) == 0
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


def test_noalloc_as_first_call_into_the_library():
    """A caller that cannot allocate may well make this its very first call: nothing else has initialised
    the library, its status word or any kernel attribute.  Runs in a fresh process and compares against a
    plain PyTorch fp32 attention computed there."""
    code = textwrap.dedent("""
        import ctypes, math, torch
        from nkipy_b200.ops import _build
        lib = ctypes.CDLL(str(_build.LIB_PATH))            # no nkb_init, no other entry point before
        P, I = ctypes.c_void_p, ctypes.c_int
        fn = lib.nkb_paged_attn_decode_noalloc
        fn.restype = I
        fn.argtypes = [P, P, P, P, P, P, I, I, I, I, I, I, I, I, ctypes.c_float, I, P, I, P]
        B, nq, nkv, D, ctx = 4, 8, 2, 128, 500
        pages = (ctx + 31) // 32
        torch.manual_seed(0)
        kc = torch.randn(B * pages, nkv, 32, D, device="cuda").to(torch.bfloat16)
        vc = torch.randn(B * pages, nkv, 32, D, device="cuda").to(torch.bfloat16)
        table = torch.arange(B * pages, device="cuda", dtype=torch.int32).reshape(B, pages)
        lens = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
        q = torch.randn(B, nq * D, device="cuda").to(torch.bfloat16)
        out = torch.empty_like(q)
        scale = 1.0 / math.sqrt(D)
        for _ in range(2):
            rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), lens.data_ptr(), out.data_ptr(),
                    B, 1, nq, nkv, D, 32, kc.shape[0], table.stride(0), scale, 0, None, 4,
                    torch.cuda.current_stream().cuda_stream)
            assert rc == 0, rc
        torch.cuda.synchronize()
        lib.nkb_noalloc_status.restype = I
        lib.nkb_noalloc_status.argtypes = [I]
        assert lib.nkb_noalloc_status(1) == 0
        k = kc.float().reshape(B, pages, nkv, 32, D).permute(0, 2, 1, 3, 4).reshape(B, nkv, pages * 32, D)[:, :, :ctx]
        v = vc.float().reshape(B, pages, nkv, 32, D).permute(0, 2, 1, 3, 4).reshape(B, nkv, pages * 32, D)[:, :, :ctx]
        qq = q.float().reshape(B, nkv, nq // nkv, D)
        p = torch.softmax(torch.einsum("bhgd,bhkd->bhgk", qq, k) * scale, dim=-1)
        ref = torch.einsum("bhgk,bhkd->bhgd", p, v).reshape(B, nq * D)
        err = ((out.float() - ref).norm() / ref.norm()).item()
        assert err < 2e-2, err
        print("NOALLOC_FIRST_OK", err)
    """)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, cwd=root)
    assert res.returncode == 0 and "NOALLOC_FIRST_OK" in res.stdout, res.stdout + res.stderr
