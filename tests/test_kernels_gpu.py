"""Numerics of the hand-written sm_100a kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch

from nkipy_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(a, b, block=128):
    """Relative error of `a` against the reference `b`: the larger of the whole-tensor Frobenius ratio and a third
    of the worst 128 x 128 block's ratio, so that one wrong tile or row slab of a large output cannot hide in the
    total.  Also asserts that no single element is off by more than 8 % of the reference's largest magnitude."""
    a, b = a.float(), b.float()
    assert a.shape == b.shape, (a.shape, b.shape)
    total = ((a - b).norm() / (b.norm() + 1e-12)).item()
    if a.numel() == 0:
        return total
    scale = b.abs().max().item() + 1e-6
    worst_abs = (a - b).abs().max().item()
    assert worst_abs <= 0.08 * scale + 1e-3, (worst_abs, scale)
    if a.dim() >= 2 and a.numel() >= 4 * block * block:
        A, B = a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1])
        pr, pc = (-A.shape[0]) % block, (-A.shape[1]) % block
        D = torch.nn.functional.pad(A - B, (0, pc, 0, pr))
        R = torch.nn.functional.pad(B, (0, pc, 0, pr))
        shape = (D.shape[0] // block, block, D.shape[1] // block, block)
        dn = D.reshape(shape).pow(2).sum(dim=(1, 3)).sqrt()
        rn = R.reshape(shape).pow(2).sum(dim=(1, 3)).sqrt()
        floor = 0.05 * scale * block            # a block of near-zero reference values is judged against the scale
        total = max(total, (dn / (rn + floor)).max().item() / 3)
    return total


def _rope_oracle(qkv, bias, pos, tab, nq, nkv, D, qn, kn, eps):
    """fp32 from the definition: bias, per-head RMSNorm (rounded to bf16 like an unfused kernel), rotate-halves."""
    T = qkv.shape[0]
    y = qkv.float() + (bias.float() if bias is not None else 0.0)
    y = y.reshape(T, nq + 2 * nkv, D)
    q, k, v = y[:, :nq], y[:, nq:nq + nkv], y[:, nq + nkv:]

    def norm(t, w):
        if w is None:
            return t
        return (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(torch.bfloat16).float()

    q, k = norm(q, qn), norm(k, kn)
    cs = tab[pos.long()]
    c, s = cs[:, None, :D // 2], cs[:, None, D // 2:]

    def rot(t):
        x, z = t[..., :D // 2], t[..., D // 2:]
        return torch.cat([x * c - z * s, z * c + x * s], dim=-1)

    return rot(q), rot(k), v


def randn(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1000, 1280, 520), (4096, 6144, 4096)])
def test_gemm_normal(M, N, K):
    x, w = randn(M, K), randn(N, K, scale=0.05)
    y = ops.linear(x, w, swap=False)
    ref = x.float() @ w.float().T
    assert rel_err(y, ref) < 1e-2


@pytest.mark.parametrize("M,N,K", [(64, 4096, 4096), (16, 256, 128), (100, 1000, 520), (128, 6144, 4096)])
def test_gemm_swapped(M, N, K):
    x, w = randn(M, K), randn(N, K, scale=0.05)
    y = ops.linear(x, w, swap=True)
    ref = x.float() @ w.float().T
    assert rel_err(y, ref) < 1e-2


@pytest.mark.parametrize("swap,M", [(True, 64), (False, 512)])
def test_gemm_splitk_bias_residual(swap, M):
    N, K = 1024, 2048
    x, w = randn(M, K), randn(N, K, scale=0.05)
    bias, res = randn(N), randn(M, N)
    parts = ops.linear(x, w, swap=swap, splits=4, bias=bias)
    assert parts.dtype == torch.float32 and parts.shape[0] == 4
    y = ops.reduce_partials(parts, residual=res)
    ref = x.float() @ w.float().T + bias.float() + res.float()
    assert rel_err(y, ref) < 1e-2
    y2 = ops.linear(x, w, swap=swap, bias=bias, residual=res)
    assert rel_err(y2, ref) < 1e-2


@pytest.mark.parametrize("swap,M", [(True, 64), (False, 384)])
def test_gemm_gated(swap, M):
    I, K = 768, 512
    x, w = randn(M, K), randn(2 * I, K, scale=0.05)
    y = ops.linear(x, w, gated=True, swap=swap)
    g, u = x.float() @ w[:I].float().T, x.float() @ w[I:].float().T
    ref = torch.nn.functional.silu(g) * u
    assert y.shape == (M, I)
    assert rel_err(y, ref) < 1e-2


def test_rmsnorm_and_fused_add():
    rows, H = 70, 4096
    x, w, r = randn(rows, H), randn(H), randn(rows, H)
    y = ops.rmsnorm(x, w, 1e-5)
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    assert rel_err(y, ref) < 5e-3
    parts = torch.randn(3, rows, H, device=DEV)
    ro, no = ops.add_rmsnorm(None, w, residual_in=r, partials=parts, eps=1e-5)
    h = (parts.sum(0) + r.float()).to(torch.bfloat16)
    assert rel_err(ro, h) < 1e-3
    hf = h.float()
    ref2 = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    assert rel_err(no, ref2) < 5e-3


def test_silu_mul_embedding_argmax():
    gu = randn(33, 2 * 1536)
    y = ops.silu_mul(gu)
    ref = torch.nn.functional.silu(gu[:, :1536].float()) * gu[:, 1536:].float()
    assert rel_err(y, ref) < 5e-3
    yc = ops.silu_mul(gu, limit=7.0, alpha=1.702)
    g, u = gu[:, :1536].float().clamp(max=7.0), gu[:, 1536:].float().clamp(-7.0, 7.0)
    assert rel_err(yc, (u + 1) * g * torch.sigmoid(1.702 * g)) < 5e-3
    table = randn(1000, 256)
    ids = torch.randint(0, 1000, (17,), device=DEV, dtype=torch.int32)
    assert torch.equal(ops.embedding(ids, table), table[ids.long()])
    logits = randn(9, 128256)
    assert torch.equal(ops.argmax(logits).long(), logits.float().argmax(-1))
    lf = torch.randn(5, 1003, device=DEV)
    assert torch.equal(ops.argmax(lf).long(), lf.argmax(-1))


def test_router_topk_both_orders():
    logits = torch.randn(50, 128, device=DEV)
    w, e = ops.router_topk(logits, 8, "softmax_topk")
    p = torch.softmax(logits, -1)
    rw, re = p.topk(8, -1)
    rw = rw / rw.sum(-1, keepdim=True)
    assert torch.equal(e.long(), re)
    assert torch.allclose(w, rw, atol=1e-5)
    w2, e2 = ops.router_topk(logits.to(torch.bfloat16), 4, "topk_softmax")
    v, re2 = logits.to(torch.bfloat16).float().topk(4, -1)
    assert torch.allclose(w2, torch.softmax(v, -1), atol=1e-5)
    parts = torch.randn(3, 50, 128, device=DEV)
    bias = randn(128)
    w3, e3 = ops.router_topk(parts, 8, "softmax_topk", bias=bias)
    p3 = torch.softmax(parts.sum(0) + bias.float(), -1)
    rw3, re3 = p3.topk(8, -1)
    assert torch.equal(e3.long(), re3) and torch.allclose(w3, rw3 / rw3.sum(-1, keepdim=True), atol=1e-5)


def test_sampling_respects_top_k():
    logits = torch.randn(8, 5000, device=DEV)
    top = logits.topk(5, -1).indices
    for step in range(4):
        ids = ops.sample(logits, temperature=0.8, top_k=5, top_p=0.95, seed=1, step=step)
        assert all(int(ids[b]) in top[b].tolist() for b in range(8))
    greedy = ops.sample(logits, temperature=1.0, top_k=1)
    assert torch.equal(greedy.long(), logits.argmax(-1))


def _make_cache(num_blocks, nkv, D):
    k = torch.zeros(num_blocks, nkv, 32, D, device=DEV, dtype=torch.bfloat16)
    return k, torch.zeros_like(k)


def _fill_cache(B, ctx_lens, nkv, D, num_blocks):
    kc, vc = _make_cache(num_blocks, nkv, D)
    max_blocks = (max(ctx_lens) + 31) // 32
    perm = torch.randperm(num_blocks)[: B * max_blocks].reshape(B, max_blocks)
    table = perm.to(torch.int32).to(DEV)
    ks, vs = [], []
    for b in range(B):
        k, v = randn(ctx_lens[b], nkv, D), randn(ctx_lens[b], nkv, D)
        ks.append(k)
        vs.append(v)
        for t in range(ctx_lens[b]):
            pass
        nb = (ctx_lens[b] + 31) // 32
        pad = nb * 32 - ctx_lens[b]
        kp = torch.cat([k, torch.zeros(pad, nkv, D, device=DEV, dtype=k.dtype)]).reshape(nb, 32, nkv, D)
        vp = torch.cat([v, torch.zeros(pad, nkv, D, device=DEV, dtype=k.dtype)]).reshape(nb, 32, nkv, D)
        kc[table[b, :nb].long()] = kp.permute(0, 2, 1, 3)
        vc[table[b, :nb].long()] = vp.permute(0, 2, 1, 3)
    return kc, vc, table, ks, vs


def _ref_attn(q, k, v, scale, q_pos0, causal=True, window=0, sinks=None):
    return ops._ref_attention(q.float(), k.float(), v.float(), scale, q_pos0, causal, window, sinks)


@pytest.mark.parametrize("nq,nkv,D,q_len,splits", [(32, 8, 128, 1, 1), (32, 8, 128, 1, 4), (8, 2, 128, 3, 2),
                                                     (8, 8, 64, 1, 1), (4, 1, 128, 2, 0)])
def test_paged_attn_decode(nq, nkv, D, q_len, splits):
    B = 5
    ctx = [1, 33, 700, 1025, 260][:B]
    ctx = [max(c, q_len) for c in ctx]
    kc, vc, table, ks, vs = _fill_cache(B, ctx, nkv, D, 256)
    q = randn(B * q_len, nq * D)
    lens = torch.tensor(ctx, device=DEV, dtype=torch.int32)
    scale = 1 / math.sqrt(D)
    out = ops.paged_attn_decode(q, kc, vc, table, lens, scale, q_len=q_len, num_splits=splits)
    for b in range(B):
        ref = _ref_attn(q[b * q_len:(b + 1) * q_len].reshape(q_len, nq, D), ks[b], vs[b], scale, ctx[b] - q_len)
        got = out[b * q_len:(b + 1) * q_len].reshape(q_len, nq, D)
        assert rel_err(got, ref) < 2e-2, (b, ctx[b])


def test_paged_attn_decode_window_and_sinks():
    nq, nkv, D, B = 8, 2, 64, 3
    ctx = [40, 300, 129]
    kc, vc, table, ks, vs = _fill_cache(B, ctx, nkv, D, 64)
    q = randn(B, nq * D)
    sinks = torch.randn(nq, device=DEV)
    lens = torch.tensor(ctx, device=DEV, dtype=torch.int32)
    scale = 1 / math.sqrt(D)
    out = ops.paged_attn_decode(q, kc, vc, table, lens, scale, window=128, sinks=sinks, num_splits=2)
    for b in range(B):
        ref = _ref_attn(q[b:b + 1].reshape(1, nq, D), ks[b], vs[b], scale, ctx[b] - 1, True, 128, sinks)
        assert rel_err(out[b].reshape(1, nq, D), ref) < 2e-2


@pytest.mark.parametrize("nq,nkv,D", [(8, 2, 128), (4, 4, 64)])
def test_flash_attn_prefill(nq, nkv, D):
    ctx = [300, 128, 1000, 77]
    q_lens = [300, 128, 488, 77]  # third sequence has a cached prefix of 512 tokens
    B = len(ctx)
    kc, vc, table, ks, vs = _fill_cache(B, ctx, nkv, D, 128)
    total = sum(q_lens)
    q = randn(total, nq * D)
    starts = [0]
    for x in q_lens[:-1]:
        starts.append(starts[-1] + x)
    t = lambda v: torch.tensor(v, device=DEV, dtype=torch.int32)
    scale = 1 / math.sqrt(D)
    out = ops.flash_attn_prefill(q, kc, vc, table, t(starts), t(q_lens), t(ctx), scale, max_q_len=max(q_lens))
    for b in range(B):
        qs = q[starts[b]:starts[b] + q_lens[b]].reshape(q_lens[b], nq, D)
        ref = _ref_attn(qs, ks[b], vs[b], scale, ctx[b] - q_lens[b])
        got = out[starts[b]:starts[b] + q_lens[b]].reshape(q_lens[b], nq, D)
        assert rel_err(got, ref) < 2e-2, b


def test_flash_attn_prefill_noncausal_window_sinks():
    nq, nkv, D = 4, 2, 64
    ctx = [200, 333]
    B = 2
    kc, vc, table, ks, vs = _fill_cache(B, ctx, nkv, D, 64)
    q = randn(sum(ctx), nq * D)
    t = lambda v: torch.tensor(v, device=DEV, dtype=torch.int32)
    scale = 1 / math.sqrt(D)
    sinks = torch.randn(nq, device=DEV)
    o1 = ops.flash_attn_prefill(q, kc, vc, table, t([0, 200]), t(ctx), t(ctx), scale, max_q_len=333, causal=False)
    o2 = ops.flash_attn_prefill(q, kc, vc, table, t([0, 200]), t(ctx), t(ctx), scale, max_q_len=333, window=128,
                                sinks=sinks)
    s = 0
    for b in range(B):
        qs = q[s:s + ctx[b]].reshape(ctx[b], nq, D)
        assert rel_err(o1[s:s + ctx[b]].reshape(ctx[b], nq, D), _ref_attn(qs, ks[b], vs[b], scale, 0, False)) < 2e-2
        assert rel_err(o2[s:s + ctx[b]].reshape(ctx[b], nq, D),
                       _ref_attn(qs, ks[b], vs[b], scale, 0, True, 128, sinks)) < 2e-2
        s += ctx[b]


def test_rope_kv_append_matches_reference():
    T, nq, nkv, D = 37, 8, 2, 128
    W = (nq + 2 * nkv) * D
    qkv = randn(T, W)
    pos = torch.randint(0, 500, (T,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(20 * 32, device=DEV)[:T].to(torch.int32)
    slots[5] = -1                                   # a row that must not reach the cache
    tab = ops.rope_table(D, 512, 500000.0, device=DEV)
    qn, kn = randn(D), randn(D)
    keep = slots >= 0
    blk, off = (slots[keep] // 32).long(), (slots[keep] % 32).long()

    def check_cache(kc, vc, rk, rv):
        assert rel_err(kc[blk, :, off], rk[keep]) < 1e-2
        assert rel_err(vc[blk, :, off], rv[keep]) < 1e-2
        untouched = torch.ones(20, 32, dtype=torch.bool, device=DEV)
        untouched[blk, off] = False
        assert kc.permute(0, 2, 1, 3)[untouched].abs().sum().item() == 0
        assert vc.permute(0, 2, 1, 3)[untouched].abs().sum().item() == 0

    kc, vc = _make_cache(20, nkv, D)
    q = ops.rope_kv_append(qkv, pos, slots, tab, kc, vc, nq, nkv, D, q_norm_w=qn, k_norm_w=kn)
    rq, rk, rv = _rope_oracle(qkv, None, pos, tab, nq, nkv, D, qn, kn, 1e-6)
    assert rel_err(q.reshape(T, nq, D), rq) < 1e-2
    check_cache(kc, vc, rk, rv)
    # fp32 split-K partials plus a bias, no QK-norm
    parts = torch.randn(3, T, W, device=DEV)
    bias = randn(W)
    kc3, vc3 = _make_cache(20, nkv, D)
    q3 = ops.rope_kv_append(parts, pos, slots, tab, kc3, vc3, nq, nkv, D, bias=bias)
    rq, rk, rv = _rope_oracle(parts.sum(0), bias, pos, tab, nq, nkv, D, None, None, 1e-6)
    assert rel_err(q3.reshape(T, nq, D), rq) < 1e-2
    check_cache(kc3, vc3, rk, rv)


@pytest.mark.parametrize("nq,nkv,D,splits,window,qknorm", [(32, 8, 128, 0, 0, False), (8, 2, 128, 4, 0, True),
                                                           (8, 8, 64, 1, 0, False), (8, 2, 64, 2, 128, True)])
def test_rope_attn_decode_one_launch(nq, nkv, D, splits, window, qknorm):
    """RoPE + cache append inside the attention kernel: output against the fp32 definition, cache contents against
    the definition, and both against the two-launch path on the same inputs."""
    B = 6
    ctx = [1, 32, 33, 700, 1025, 260]                      # lengths that already count the new token
    kc, vc, table, ks, vs = _fill_cache(B, ctx, nkv, D, 256)
    W = (nq + 2 * nkv) * D
    parts = torch.randn(5, B, W, device=DEV) * 0.4
    bias = randn(W)
    qn, kn = (randn(D), randn(D)) if qknorm else (None, None)
    sinks = torch.randn(nq, device=DEV) if window else None
    tab = ops.rope_table(D, 2048, 500000.0, device=DEV)
    lens = torch.tensor(ctx, device=DEV, dtype=torch.int32)
    pos = lens - 1
    slots = torch.stack([table[b, (ctx[b] - 1) // 32] * 32 + (ctx[b] - 1) % 32 for b in range(B)]).to(torch.int32)
    scale = 1 / math.sqrt(D)
    kc2, vc2 = kc.clone(), vc.clone()
    out = ops.rope_attn_decode(parts, pos, slots, tab, kc, vc, table, lens, scale, nq, nkv, bias=bias, q_norm_w=qn,
                               k_norm_w=kn, window=window, sinks=sinks, num_splits=splits)
    q2 = ops.rope_kv_append(parts, pos, slots, tab, kc2, vc2, nq, nkv, D, bias=bias, q_norm_w=qn, k_norm_w=kn)
    out2 = ops.paged_attn_decode(q2, kc2, vc2, table, lens, scale, window=window, sinks=sinks, num_splits=splits)
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)     # same arithmetic, same rounding
    rq, rk, rv = _rope_oracle(parts.sum(0), bias, pos, tab, nq, nkv, D, qn, kn, 1e-6)
    for b in range(B):
        k = torch.cat([ks[b][:ctx[b] - 1].float(), rk[b:b + 1]])
        v = torch.cat([vs[b][:ctx[b] - 1].float(), rv[b:b + 1]])
        ref = _ref_attn(rq[b:b + 1], k, v, scale, ctx[b] - 1, True, window, sinks)
        assert rel_err(out[b].reshape(1, nq, D), ref) < 2e-2, (b, ctx[b])
        assert rel_err(out[b].reshape(1, nq, D), out2[b].reshape(1, nq, D).float()) < 1e-2, (b, ctx[b])
    # an inactive sequence (negative length, slot -1) writes nothing
    lens[2] = -1
    slots[2] = -1
    before = kc.clone()
    ops.rope_attn_decode(parts, pos, slots, tab, kc, vc, table, lens, scale, nq, nkv, bias=bias, q_norm_w=qn,
                         k_norm_w=kn, window=window, sinks=sinks, num_splits=splits)
    torch.cuda.synchronize()
    assert torch.equal(kc[table[2, 1].long()], before[table[2, 1].long()])


def test_decode_advance():
    B = 4
    ctx = torch.tensor([5, 31, 32, -1], device=DEV, dtype=torch.int32)
    table = torch.arange(B * 3, device=DEV, dtype=torch.int32).reshape(B, 3) + 10
    pos = torch.empty(B, device=DEV, dtype=torch.int32)
    slots = torch.empty(B, device=DEV, dtype=torch.int32)
    ops.decode_advance(ctx, table, pos, slots)
    assert pos.tolist() == [5, 31, 32, 0]
    assert slots.tolist() == [10 * 32 + 5, 13 * 32 + 31, 17 * 32 + 0, -1]
    assert ctx.tolist() == [6, 32, 33, -1]


def test_silu_mul_from_split_partials():
    T, I = 48, 1792
    parts = torch.randn(3, T, 2 * I, device=DEV)
    bias = randn(2 * I)
    y = ops.silu_mul(parts, bias=bias)
    x = parts.sum(0) + bias.float()
    ref = torch.nn.functional.silu(x[:, :I]) * x[:, I:]
    assert rel_err(y, ref) < 5e-3
    yc = ops.silu_mul(parts, limit=7.0)
    x = parts.sum(0)
    g, u = x[:, :I].clamp(max=7.0), x[:, I:].clamp(-7.0, 7.0)
    assert rel_err(yc, (u + 1) * g * torch.sigmoid(1.702 * g)) < 5e-3


@pytest.mark.parametrize("T,E,k,H,I,lo,nl", [(128, 16, 4, 512, 256, 0, 16), (37, 8, 2, 256, 128, 4, 4),
                                              (300, 8, 2, 256, 384, 0, 8)])
def test_moe_dispatch_grouped_gemm_combine(T, E, k, H, I, lo, nl):
    x = randn(T, H)
    logits = torch.randn(T, E, device=DEV)
    wts, experts = ops.router_topk(logits, k, "softmax_topk")
    xs, off, pos = ops.moe_dispatch(x, experts, lo, nl)
    xs_c, off_c, pos_c = ops.moe_dispatch(x.cpu(), experts.cpu(), lo, nl)
    assert torch.equal(off.cpu(), off_c)
    n_local = int(off_c[-1])
    assert ((pos.cpu() >= 0) == (pos_c >= 0)).all() and int((pos >= 0).sum()) == n_local
    # rows land in the right expert segment and carry the right token
    flat_e = experts.reshape(-1).cpu() - lo
    for p in range(T * k):
        if pos[p] >= 0:
            e = int(flat_e[p])
            assert off_c[e] <= int(pos[p]) < off_c[e + 1]
    sel = (pos >= 0).nonzero().squeeze(-1)
    assert torch.equal(xs[pos[sel].long()], x[(sel // k)])
    w_gu = randn(nl, 2 * I, H, scale=0.05)
    w_dn = randn(nl, H, I, scale=0.05)
    b_gu, b_dn = randn(nl, 2 * I, scale=0.1), randn(nl, H, scale=0.1)
    plan = ops.moe_dispatch(x, experts, lo, nl)
    h = ops.grouped_linear(plan.x_sorted, w_gu, plan.offsets, max_rows_per_group=T, gated=True, bias=b_gu,
                           tiles=plan.tiles)
    y = ops.grouped_linear(h, w_dn, plan.offsets, max_rows_per_group=T, bias=b_dn, tiles=plan.tiles)
    pos, off = plan.pair_pos, plan.offsets
    h2 = ops.grouped_linear(plan.x_sorted, w_gu, off, max_rows_per_group=T, gated=True, bias=b_gu)   # enumerated schedule
    assert rel_err(h2[:n_local], h[:n_local]) < 1e-3
    out = ops.moe_combine(y, pos, wts, T)
    # fp32 reference straight from the definition
    ref = torch.zeros(T, H, device=DEV)
    for t in range(T):
        for j in range(k):
            e = int(experts[t, j]) - lo
            if 0 <= e < nl:
                z = x[t].float() @ w_gu[e].float().T + b_gu[e].float()
                a = torch.nn.functional.silu(z[:I]) * z[I:]
                ref[t] += wts[t, j] * (a.to(torch.bfloat16).float() @ w_dn[e].float().T + b_dn[e].float())
    assert rel_err(out, ref) < 2e-2
    hc = ops.grouped_linear(xs, w_gu, off, max_rows_per_group=T, gated=True, act_limit=7.0, act_alpha=1.702)
    # clamped SwiGLU from its definition: gate <= limit, |up| <= limit, (up + 1) * gate * sigmoid(alpha * gate)
    offs = off.cpu().tolist()
    hc_ref = torch.zeros(n_local, I, device=DEV)
    for e in range(nl):
        rows = slice(offs[e], offs[e + 1])
        z = xs[rows].float() @ w_gu[e].float().T
        g, u = z[:, :I].clamp(max=7.0), z[:, I:].clamp(-7.0, 7.0)
        hc_ref[rows] = (u + 1) * g * torch.sigmoid(1.702 * g)
    assert rel_err(hc[:n_local], hc_ref) < 2e-2


@pytest.mark.parametrize("M,N,K,bias,resid", [(512, 256, 64, False, False), (1024, 768, 512, True, True),
                                              (640, 392, 192, True, False), (2048, 1024, 1024, False, True)])
def test_linear_cta_pair_kernel(M, N, K, bias, resid):
    """Prefill-sized GEMMs take the cta_group::2 kernel (256 x 256 tiles on CTA pairs); ragged edges included."""
    import nkipy_b200.ops as O

    assert O._USE_2CTA
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(M + N)
    x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, device=dev, generator=g).to(torch.bfloat16) if bias else None
    r = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16) if resid else None
    y = O.linear(x, w, bias=b, residual=r, swap=False)
    assert O._lib.lib().nkb_gemm_2cta_pairs() > 0          # the pair kernel really ran
    ref = x.float() @ w.float().T
    if b is not None:
        ref += b.float()
    if r is not None:
        ref += r.float()
    rel = ((y.float() - ref).norm() / ref.norm()).item()
    assert rel < 5e-3, rel
    assert O.device_status() == 0


@pytest.mark.parametrize("M,I,K", [(512, 256, 128), (1024, 1408, 512), (640, 392, 192)])
def test_linear_cta_pair_kernel_gated(M, I, K):
    """SwiGLU on CTA pairs: the first CTA of a pair loads gate rows, the second up rows."""
    import nkipy_b200.ops as O

    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(M + I)
    x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    y = O.linear(x, w, gated=True, swap=False)
    ref = torch.nn.functional.silu(x.float() @ w[:I].float().T) * (x.float() @ w[I:].float().T)
    rel = ((y.float() - ref).norm() / ref.norm()).item()
    assert y.shape == (M, I) and rel < 1e-2, rel
    assert O.device_status() == 0
