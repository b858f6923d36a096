"""Decode GEMMs that finish their own split-K sum -- the last-arriver fix-up inside the persistent GEMM
(csrc/kernels/splitk_fix.cuh) and the cluster / distributed-shared-memory variant
(csrc/kernels/gemm_decode.cu) -- against fp32 PyTorch oracles written here.

Besides the whole-tensor relative error every comparison checks each 128-column block of the output on its
own and the largest absolute deviation, so that one wrong tile (or one wrong cluster rank's token slice)
cannot hide inside a large tensor.
"""
import math

import pytest
import torch

from nkipy_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def randn(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(torch.bfloat16)


def check(out, ref, tol=1e-2, block=128):
    out, ref = out.float(), ref.float()
    assert out.shape == ref.shape
    assert torch.isfinite(out).all()
    total = ((out - ref).norm() / (ref.norm() + 1e-12)).item()
    assert total < tol, total
    scale = ref.abs().max().item() + 1e-6
    assert (out - ref).abs().max().item() < 0.05 * scale
    flat_o, flat_r = out.reshape(out.shape[0], -1), ref.reshape(ref.shape[0], -1)
    for c in range(0, flat_o.shape[1], block):
        for r in range(0, flat_o.shape[0], 8):
            o, rr = flat_o[r:r + 8, c:c + block], flat_r[r:r + 8, c:c + block]
            e = ((o - rr).norm() / (rr.norm() + 1e-3 * scale)).item()
            assert e < 3 * tol, (r, c, e)


IMPLS = ["fixup", "cluster"]


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("M,N,K,S", [(64, 4096, 512, 4), (17, 768, 4096, 8), (128, 2048, 4096, 2), (64, 1000, 1792, 8),
                                     (1, 256, 128, 1), (32, 4096, 4096, 8), (100, 512, 64, 4), (64, 6144, 4096, 6),
                                     (64, 4096, 14336, 3)])
def test_decode_linear_matches_fp32(M, N, K, S, impl):
    x, w = randn(M, K), randn(N, K, scale=0.05)
    y = ops.decode_linear(x, w, splits=S, impl=impl)
    check(y, x.float() @ w.float().T)
    assert ops.device_status() == 0


@pytest.mark.parametrize("impl", IMPLS)
def test_decode_linear_bias_residual(impl):
    M, N, K = 48, 1536, 2048
    x, w, b, r = randn(M, K), randn(N, K, scale=0.05), randn(N), randn(M, N)
    y = ops.decode_linear(x, w, splits=4, bias=b, residual=r, impl=impl)
    check(y, x.float() @ w.float().T + b.float() + r.float())


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("M,I,K,S", [(64, 1792, 4096, 8), (128, 768, 2048, 4), (20, 14336, 4096, 1), (64, 96, 256, 2)])
def test_decode_linear_swiglu(M, I, K, S, impl):
    x, w = randn(M, K), randn(2 * I, K, scale=0.05)
    y = ops.decode_linear(x, w, splits=S, gated=True, impl=impl)
    g, u = x.float() @ w[:I].float().T, x.float() @ w[I:].float().T
    check(y, torch.nn.functional.silu(g) * u)
    assert y.shape == (M, I)


@pytest.mark.parametrize("impl", IMPLS)
def test_decode_linear_clamped_swiglu_with_bias(impl):
    M, I, K = 24, 640, 1024
    x, w, b = randn(M, K), randn(2 * I, K, scale=0.1), randn(2 * I)
    lim, alpha = 7.0, 1.702
    y = ops.decode_linear(x, w, splits=4, gated=True, bias=b, act_limit=lim, act_alpha=alpha, impl=impl)
    g = (x.float() @ w[:I].float().T + b[:I].float()).clamp(max=lim)
    u = (x.float() @ w[I:].float().T + b[I:].float()).clamp(-lim, lim)
    check(y, (u + 1) * g * torch.sigmoid(alpha * g))


def _qkv_oracle(x, w, bias, pos, cos_sin, nq, nkv, D, qn, kn, eps):
    """fp32: projection, per-head RMSNorm (rounded to bf16 like an unfused kernel), rotate-halves RoPE."""
    T = x.shape[0]
    y = x.float() @ w.float().T
    if bias is not None:
        y = y + bias.float()
    y = y.reshape(T, nq + 2 * nkv, D)
    q, k, v = y[:, :nq], y[:, nq:nq + nkv], y[:, nq + nkv:]

    def norm(t, wt):
        if wt is None:
            return t
        return (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * wt.float()).to(torch.bfloat16).float()

    q, k = norm(q, qn), norm(k, kn)
    cs = cos_sin[pos.long()]
    c, s = cs[:, None, :D // 2], cs[:, None, D // 2:]

    def rot(t):
        a, b = t[..., :D // 2], t[..., D // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

    return rot(q), rot(k), v


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("T,nq,nkv,D,K,S,norm,use_bias", [
    (64, 4, 1, 128, 4096, 8, False, False),      # Llama shard of 8
    (128, 32, 4, 128, 2048, 2, True, False),     # Qwen3 with QK-norm
    (40, 8, 2, 64, 1024, 4, False, True),        # head_dim 64 with bias
    (9, 6, 2, 64, 512, 2, True, True),
])
def test_qkv_rope_append_matches_oracle(T, nq, nkv, D, K, S, norm, use_bias, impl):
    torch.manual_seed(T + nq)
    x, w = randn(T, K), randn((nq + 2 * nkv) * D, K, scale=0.05)
    bias = randn((nq + 2 * nkv) * D) if use_bias else None
    qn = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16) if norm else None
    kn = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16) if norm else None
    max_pos, bs, nblocks = 512, 32, 12
    cos_sin = ops.rope_table(D, max_pos, theta=10000.0, device=DEV)
    pos = torch.randint(0, max_pos, (T,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(nblocks * bs, device=DEV)[:T].to(torch.int32)
    slots[T // 2] = -1                      # a row that must not be stored
    kc = torch.zeros(nblocks, nkv, bs, D, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q = ops.qkv_rope_append(x, w, pos, slots, cos_sin, kc, vc, nq, nkv, D, splits=S, bias=bias, q_norm_w=qn,
                            k_norm_w=kn, norm_eps=1e-6, impl=impl)
    rq, rk, rv = _qkv_oracle(x, w, bias, pos, cos_sin, nq, nkv, D, qn, kn, 1e-6)
    check(q.reshape(T, nq, D), rq, tol=1.5e-2)
    keep = slots >= 0
    blk, off = (slots[keep] // bs).long(), (slots[keep] % bs).long()
    check(kc[blk, :, off], rk[keep], tol=1.5e-2)
    check(vc[blk, :, off], rv[keep], tol=1.5e-2)
    # nothing but the addressed slots was written
    mask = torch.ones(nblocks, bs, dtype=torch.bool, device=DEV)
    mask[blk, off] = False
    assert kc.permute(0, 2, 1, 3)[mask].abs().sum().item() == 0
    assert vc.permute(0, 2, 1, 3)[mask].abs().sum().item() == 0
    assert ops.device_status() == 0


@pytest.mark.parametrize("impl", IMPLS)
def test_decode_linear_back_to_back_launches_share_scratch(impl):
    """Programmatic dependent launch lets consecutive kernels overlap, and the fix-up launches share one
    partial buffer and one set of counters per stream; results must not depend on either."""
    M, K = 64, 2048
    x = randn(M, K)
    ws = [randn(1024, K, scale=0.05) for _ in range(6)]
    outs = [ops.decode_linear(x, w, splits=4, impl=impl) for w in ws]
    for w, y in zip(ws, outs):
        check(y, x.float() @ w.float().T)
