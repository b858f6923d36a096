"""Single-kernel micro-benchmarks of the sm_100a kernel library.

    python -m nkipy_b200.ops.microbench <case> [--iters N] [--sets S]

Each case launches one kernel of the library at a serving shape, rotating over several
operand sets so that every launch reads data that is not in L2 (the sets together exceed
the 126 MB cache), times the launches with CUDA events after warm-up and prints one JSON
line: microseconds per launch, algorithmic bytes and FLOPs, achieved TB/s and TFLOP/s and
their fraction of the measured peaks (``MEASURED_PEAKS.json`` beside the package when it
exists, otherwise 6.65 TB/s and 1590 TFLOP/s).  The same command line is what the profiler
is pointed at (``--iters 1 --warmup 1`` keeps a capture short).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from . import (add_rmsnorm, decode_linear, flash_attn_prefill, grouped_linear, linear, moe_combine, moe_dispatch,
               paged_attn_decode, router_topk)

_FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return dict(_FALLBACK, source="fallback")


def _bf16(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _time(fns, iters, warmup, graph=True):
    """fns: list of callables (one per operand set); returns us per launch.  With graph=True one
    pass over all sets is captured into a CUDA graph and replayed, so that host launch cost does
    not hide the device time of kernels that run for a few microseconds."""
    n = len(fns)
    for i in range(max(warmup, 1)):
        fns[i % n]()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for f in fns:
                f()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for f in fns:
                f()
        reps = max(1, iters // n)
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (reps * n)
    e0.record()
    for i in range(iters):
        fns[i % n]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def _sets_for(bytes_per_set, want):
    # enough sets that a rotation touches > 2x L2 between two uses of the same set
    need = int(2 * 126e6 / max(bytes_per_set, 1)) + 1
    return max(2, min(max(need, 2), want))


# --------------------------------------------------------------------------- cases
def case_gemm_decode(name, features, k, tokens, splits, gated, args, row_parallel=False):
    """One decode projection.  --impl splitk: the persistent GEMM (fp32 split-K partials left to the next
    kernel); --impl cluster: the cluster GEMM that sums the splits through distributed shared memory and
    applies the epilogue itself.  --tp N takes the per-rank shard of an N-way tensor-parallel layer."""
    if args.splits > 0 and (not gated or args.impl != "splitk"):
        splits = args.splits
    if args.tokens > 0:
        tokens = args.tokens
    if args.tp > 1:
        if row_parallel:
            k //= args.tp
        else:
            features //= args.tp
    wrows = features * (2 if gated else 1)
    nbytes = wrows * k * 2
    sets = _sets_for(nbytes, max(args.sets, 2))
    ws = [_bf16(wrows, k, scale=0.02) for _ in range(sets)]
    x = _bf16(tokens, k)
    if args.impl in ("cluster", "fixup"):
        fns = [lambda w=w: decode_linear(x, w, splits=splits, gated=gated, impl=args.impl) for w in ws]
        out_bytes = tokens * features * 2
    else:
        fns = [lambda w=w: linear(x, w, splits=splits, gated=gated) for w in ws]
        out_bytes = tokens * features * (4 * splits if splits > 1 else 2)
    us = _time(fns, args.iters, args.warmup, not args.no_graph)
    return dict(case=name, us=us, bytes=nbytes + tokens * k * 2 + out_bytes,
                flops=2.0 * tokens * wrows * k, shape=dict(features=features, k=k, tokens=tokens, splits=splits,
                                                           gated=gated, sets=sets, impl=args.impl, tp=args.tp))


def case_gemm_decode_sweep(args):
    """Both implementations of the four decode projections of Llama-3-8B at tp = 1 and tp = 8 over a range of
    split factors; prints one compact line per point (us per launch and fraction of the measured copy
    bandwidth) and returns the last point."""
    import copy

    pk = peaks()
    last = None
    shapes = [("qkv", 6144, 4096, False, False), ("o", 4096, 4096, False, True),
              ("gate-up", 14336, 4096, True, False), ("down", 4096, 14336, False, True)]
    for tp in (1, 8):
        for nm, feat, k, gated, rowp in shapes:
            for impl in ("splitk", "fixup", "cluster"):
                cands = (2, 4, 8) if impl == "cluster" else ((1,) if gated and impl == "splitk" else (1, 4, 6, 8))
                for sp in cands:
                    a = copy.copy(args)
                    a.impl, a.tp, a.splits, a.tokens = impl, tp, sp, 64
                    torch.manual_seed(0)
                    try:
                        r = case_gemm_decode(f"gemm-decode-{nm}", feat, k, 64, sp, gated, a, rowp)
                    except Exception as e:  # noqa: BLE001 - a rejected configuration is reported, not fatal
                        print(json.dumps(dict(case=nm, tp=tp, impl=impl, splits=sp, error=str(e)[:120])), flush=True)
                        continue
                    frac = r["bytes"] / r["us"] / 1e6 * 1e3 / pk["hbm_gbs"]
                    print(json.dumps(dict(case=nm, tp=tp, impl=impl, splits=sp, us=round(r["us"], 2),
                                          frac_hbm=round(frac, 3))), flush=True)
                    last = r
                    torch.cuda.empty_cache()
    return last


def case_gemm_prefill(args):
    M, K, N = 8192, 4096, 14336
    x = _bf16(M, K)
    ws = [_bf16(N, K, scale=0.02) for _ in range(2)]
    fns = [lambda w=w: linear(x, w) for w in ws]
    us = _time(fns, args.iters, args.warmup, not args.no_graph)
    return dict(case="gemm-prefill", us=us, bytes=(M * K + N * K + M * N) * 2, flops=2.0 * M * N * K,
                shape=dict(M=M, K=K, N=N))


def case_gemm_prefill_gated(args):
    M, K, I = 8192, 4096, 14336
    x = _bf16(M, K)
    ws = [_bf16(2 * I, K, scale=0.02) for _ in range(2)]
    fns = [lambda w=w: linear(x, w, gated=True, swap=False) for w in ws]
    us = _time(fns, args.iters, args.warmup, not args.no_graph)
    return dict(case="gemm-prefill-gated", us=us, bytes=(M * K + 2 * I * K + M * I) * 2, flops=4.0 * M * I * K,
                shape=dict(M=M, K=K, I=I, note="gate/up GEMM with the SwiGLU epilogue on CTA pairs"))


def case_gemm_comm(mode, args):
    """The fused GEMM + collective kernels with a single rank: same tcgen05 pipeline, staging / pusher paths
    included, no NVLink traffic (multi-GPU numbers come from bench_fused.py)."""
    from ..parallel.comm import TPGroup
    from ..parallel.symm import AllGatherGemm, GemmReduceScatter

    tp = TPGroup.single(torch.device("cuda"))
    if mode == "rs":
        M, K, N = 8192, 4096, 8192
        op = GemmReduceScatter(tp, M, N)
    else:
        M, K, N = 8192, 8192, 3584               # one rank: every tile is local, no pusher CTA is needed
        op = AllGatherGemm(tp, M, K)
    x = _bf16(M, K)
    ws = [_bf16(N, K, scale=0.02) for _ in range(2)]
    fns = [lambda w=w: op(x, w) for w in ws]
    us = _time(fns, args.iters, args.warmup, False)
    r = dict(case=f"gemm-{mode}-tp1" if mode == "rs" else "ag-gemm-tp1", us=us, bytes=(M * K + N * K + M * N) * 2,
             flops=2.0 * M * N * K, shape=dict(M=M, K=K, N=N, ranks=1))
    torch.cuda.synchronize()
    op.close()
    return r


def case_gemm_ar(args):
    """Decode-form row-parallel GEMM whose epilogue stores its partial tiles into the symmetric buffers, followed
    by the consumer (wait on the arrival counters, sum, residual, RMSNorm); one rank, so no NVLink traffic."""
    from ..parallel.comm import TPGroup
    from ..parallel.symm import FusedTP

    M, K, N = 64, 14336, 4096                     # Llama-3-8B down projection at batch 64
    fused = FusedTP(TPGroup.single(torch.device("cuda")), M, N)
    x = _bf16(M, K)
    resid, wn = _bf16(M, N), _bf16(N)
    sets = _sets_for(N * K * 2, args.sets)
    sets += sets % 2                              # the two partial buffers alternate per call
    ws = [_bf16(N, K, scale=0.02) for _ in range(sets)]
    fns = [lambda w=w: fused.gemm_allreduce_add_rmsnorm(x, w, resid, wn, None, 1e-5, splits=8) for w in ws]
    us = _time(fns, args.iters, args.warmup, not args.no_graph)
    r = dict(case="gemm-ar-tp1", us=us, bytes=(M * K + N * K + 3 * M * N) * 2, flops=2.0 * M * N * K,
             shape=dict(M=M, K=K, N=N, ranks=1, sets=sets, launches_per_call=2))
    torch.cuda.synchronize()
    fused.close()
    return r


def case_attn_decode(args):
    B, ctx, nkv, nq, D = 64, 1056, 8, 32, 128
    if args.tp > 1:                       # one rank's heads of an N-way tensor-parallel layer
        nkv, nq = max(1, nkv // args.tp), nq // args.tp
    pages = (ctx + 31) // 32
    nb = B * pages
    per_set = 2 * nb * nkv * 32 * D * 2
    sets = _sets_for(per_set, args.sets)
    caches = [(_bf16(nb, nkv, 32, D), _bf16(nb, nkv, 32, D)) for _ in range(sets)]
    table = torch.arange(nb, device="cuda", dtype=torch.int32).reshape(B, pages)
    lens = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
    q = _bf16(B, nq * D)
    fns = [lambda kc=kc, vc=vc: paged_attn_decode(q, kc, vc, table, lens, D ** -0.5, num_splits=args.kv_splits)
           for kc, vc in caches]
    us = _time(fns, args.iters, args.warmup, not args.no_graph)
    return dict(case="attn-decode", us=us, bytes=B * ctx * nkv * D * 2 * 2, flops=4.0 * B * nq * ctx * D,
                shape=dict(batch=B, context=ctx, nq=nq, nkv=nkv, head_dim=D, sets=sets, kv_splits=args.kv_splits))


def case_attn_prefill(args):
    B, S, nq, nkv, D = args.batch or 8, args.seq or 2048, 32, 8, 128
    pages = S // 32
    nb = B * pages
    kc, vc = _bf16(nb, nkv, 32, D), _bf16(nb, nkv, 32, D)
    table = torch.arange(nb, device="cuda", dtype=torch.int32).reshape(B, pages)
    q = _bf16(B * S, nq * D)
    q_start = torch.arange(B, device="cuda", dtype=torch.int32) * S
    q_lens = torch.full((B,), S, device="cuda", dtype=torch.int32)
    fns = [lambda: flash_attn_prefill(q, kc, vc, table, q_start, q_lens, q_lens, D ** -0.5, max_q_len=S, causal=True)]
    us = _time(fns, args.iters, args.warmup, not args.no_graph)
    return dict(case="attn-prefill", us=us, bytes=(2 * q.numel() + kc.numel() + vc.numel()) * 2,
                flops=4.0 * B * nq * S * S * D / 2, shape=dict(batch=B, seq=S, nq=nq, nkv=nkv, head_dim=D, causal=True))


def case_moe(args):
    """The grouped expert GEMMs of one Qwen3-30B-A3B decode layer (128 tokens, top-8 of 128 experts)."""
    T, H, E, I, topk = 128, 2048, 128, 768, 8
    sets = max(2, min(args.sets, 4))
    w13 = [_bf16(E, 2 * I, H, scale=0.02) for _ in range(sets)]
    w2 = [_bf16(E, H, I, scale=0.02) for _ in range(sets)]
    x = _bf16(T, H)
    logits = torch.randn(T, E, device="cuda")
    wts, experts = router_topk(logits, topk)

    def layer(a, b):
        plan = moe_dispatch(x, experts, 0, E)
        h = grouped_linear(plan.x_sorted, a, plan.offsets, max_rows_per_group=T, gated=True, tiles=plan.tiles)
        y = grouped_linear(h, b, plan.offsets, max_rows_per_group=T, tiles=plan.tiles)
        return moe_combine(y, plan.pair_pos, wts, T)

    fns = [lambda a=a, b=b: layer(a, b) for a, b in zip(w13, w2)]
    us = _time(fns, args.iters, args.warmup, not args.no_graph)
    return dict(case="moe-decode-layer", us=us, bytes=E * 3 * I * H * 2, flops=2.0 * T * topk * 3 * I * H,
                shape=dict(tokens=T, hidden=H, experts=E, inter=I, top_k=topk, sets=sets,
                           note="dispatch + gated grouped GEMM + down grouped GEMM + combine; bytes = all expert weights"))


def case_moe_push(args):
    """The expert-parallel MoE block as a rank runs it (router, dispatch, two grouped GEMMs, the combine kernel
    that stores every token's weighted partial sum into the peers' buffers, the summing residual + RMSNorm
    kernel) with one rank, i.e. without NVLink traffic."""
    from ..models import config as C
    from ..models.moe import MoEBlock
    from ..parallel.comm import TPGroup
    from ..parallel.symm import FusedTP

    cfg = C.qwen3_30b_a3b()
    T, H, E, I = 128, cfg.hidden_size, cfg.num_experts, cfg.moe_intermediate_size
    tp = TPGroup.single(torch.device("cuda"))
    fused = FusedTP(tp, T, H)
    blk = MoEBlock(cfg, tp, "ep")
    sets = max(2, min(args.sets, 4))
    sets += sets % 2

    class LW:
        router_bias = gate_up_bias = down_bias = None

    lws = []
    for _ in range(sets):
        lw = LW()
        lw.router, lw.gate_up, lw.down = _bf16(E, H, scale=0.02), _bf16(E, 2 * I, H, scale=0.02), _bf16(E, H, I, scale=0.02)
        lws.append(lw)
    x, resid, wn = _bf16(T, H), _bf16(T, H), _bf16(H)

    def layer(lw):
        y_sorted, plan, weights = blk._experts(lw, x)
        return fused.moe_combine_allreduce_add_rmsnorm(y_sorted, plan.pair_pos, weights, T, resid, wn, cfg.rms_eps)

    fns = [lambda lw=lw: layer(lw) for lw in lws]
    us = _time(fns, args.iters, args.warmup, not args.no_graph)
    r = dict(case="moe-ep-block-tp1", us=us, bytes=E * 3 * I * H * 2, flops=2.0 * T * cfg.top_k * 3 * I * H,
             shape=dict(tokens=T, hidden=H, experts=E, inter=I, top_k=cfg.top_k, ranks=1, sets=sets))
    torch.cuda.synchronize()
    fused.close()
    return r


def case_addnorm(args):
    T, H, S = 64, 4096, 8
    parts = [torch.randn(S, T, H, device="cuda") for _ in range(4)]
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    r = _bf16(T, H)
    fns = [lambda p=p: add_rmsnorm(None, w, residual_in=r, partials=p, eps=1e-5) for p in parts]
    us = _time(fns, args.iters, args.warmup, not args.no_graph)
    return dict(case="add-rmsnorm", us=us, bytes=S * T * H * 4 + 3 * T * H * 2, flops=0.0,
                shape=dict(tokens=T, hidden=H, splits=S))


def case_decode_layer(args):
    """One launch of the persistent decode-layer kernel at Llama-3-8B shapes (the per-rank shard with --tp N),
    rotating over enough weight sets to exceed L2; `stages_us` are CTA 0's global-timer intervals per stage
    (o_proj, reduce, gate/up, [silu], down, reduce, qkv, rope + exit), averaged over the sets."""
    from . import decode_layer as DL
    from . import rope_table

    tp = max(1, args.tp)
    T, H, D = (args.tokens or 64), 4096, 128
    nq, nkv, inter = 32 // tp, max(1, 8 // tp), 14336 // tp
    k_o, qkv_w = nq * D, (nq + 2 * nkv) * D
    per_set = 2 * (H * k_o + 2 * inter * H + H * inter + qkv_w * H)
    sets = _sets_for(per_set, args.sets)
    fused_gate = inter // 128 >= 100
    env = DL.env_splits() or (0, 0, 0, 0)
    pick = DL.pick_layer_splits
    sp = [pick(H, k_o), 1 if fused_gate else pick(2 * inter, H), pick(H, inter), pick(qkv_w, H)]
    sp = [e if e > 0 else d for e, d in zip(env, sp)]
    if sp[1] > 1:
        fused_gate = False
    scratch = DL.layer_scratch("cuda", DL.scratch_floats(DL.block_n_for(T), [
        (H, sp[0]), (0 if fused_gate else 2 * inter, sp[1]), (H, sp[2]), (qkv_w, sp[3])]))
    cos_sin = rope_table(D, 4096, theta=500000.0, device="cuda")
    pos = torch.randint(0, 4096, (T,), device="cuda", dtype=torch.int32)
    slots = torch.arange(T, device="cuda", dtype=torch.int32)
    bs = 32
    kc = torch.zeros((T + bs - 1) // bs + 1, nkv, bs, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    mask = DL.ST_ALL if not fused_gate else DL.ST_ALL & ~DL.ST_SILU
    timings, fns = [], []
    for _ in range(sets):
        w = dict(w_o=_bf16(H, k_o, scale=0.02), w_gu=_bf16(2 * inter, H, scale=0.02), w_down=_bf16(H, inter, scale=0.02),
                 w_qkv=_bf16(qkv_w, H, scale=0.02))
        io = dict(attn=_bf16(T, k_o), resid_in=_bf16(T, H), norm1_w=_bf16(H), norm2_w=_bf16(H),
                  resid_mid=_bf16(T, H), normed_mid=_bf16(T, H), act=_bf16(T, inter), resid_out=_bf16(T, H),
                  normed_out=_bf16(T, H), q_out=_bf16(T, nq * D))
        tm = torch.zeros(80, dtype=torch.int64, device="cuda")
        timings.append(tm)

        def fn(w=w, io=io, tm=tm):
            DL.decode_layer(mask, T, H, 1e-5, scratch, splits_o=sp[0], inter=inter, splits_gu=sp[1],
                            fused_gate=fused_gate, splits_down=sp[2], splits_qkv=sp[3], nq=nq, nkv=nkv, head_dim=D,
                            positions=pos, slots=slots, cos_sin=cos_sin, k_cache=kc, v_cache=vc, timing=tm, **w, **io)
        fns.append(fn)
    us = _time(fns, args.iters, args.warmup, graph=not args.no_graph)
    torch.cuda.synchronize()
    n_stage = bin(mask).count("1")
    raw = torch.stack(timings).double().cpu()
    ticks = raw[:, :n_stage + 1]
    stages = (ticks[:, 1:] - ticks[:, :-1]).mean(0) / 1e3
    # phases of the four GEMM stages relative to each stage's entry
    phases = []
    for g in range(4):
        m = raw[:, 16 + 16 * g:32 + 16 * g]
        phases.append([round(float(x), 2) for x in ((m - m[:, :1]).mean(0) / 1e3)])
    return dict(case="decode-layer", tp=tp, tokens=T, splits=sp, fused_gate=fused_gate, sets=sets, us=us,
                bytes=per_set, flops=2.0 * T * per_set / 2, stages_us=[round(float(x), 2) for x in stages],
                gemm_phases_us=phases)


CASES = {
    "decode-layer": case_decode_layer,
    "gemm-decode-qkv": lambda a: case_gemm_decode("gemm-decode-qkv", 6144, 4096, 64, 6, False, a),
    "gemm-decode-o": lambda a: case_gemm_decode("gemm-decode-o", 4096, 4096, 64, 8, False, a, True),
    "gemm-decode-gate-up": lambda a: case_gemm_decode("gemm-decode-gate-up", 14336, 4096, 64, 1, True, a),
    "gemm-decode-down": lambda a: case_gemm_decode("gemm-decode-down", 4096, 14336, 64, 8, False, a, True),
    "gemm-decode-sweep": case_gemm_decode_sweep,
    "gemm-decode-lmhead": lambda a: case_gemm_decode("gemm-decode-lmhead", 128256, 4096, 64, 1, False, a),
    "gemm-prefill": case_gemm_prefill,
    "gemm-prefill-gated": case_gemm_prefill_gated,
    "gemm-rs-tp1": lambda a: case_gemm_comm("rs", a),
    "ag-gemm-tp1": lambda a: case_gemm_comm("ag", a),
    "gemm-ar-tp1": case_gemm_ar,
    "attn-decode": case_attn_decode,
    "attn-prefill": case_attn_prefill,
    "moe-decode-layer": case_moe,
    "moe-ep-block-tp1": case_moe_push,
    "add-rmsnorm": case_addnorm,
}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=sorted(CASES) + ["all"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--sets", type=int, default=8, help="upper bound of rotating operand sets")
    ap.add_argument("--splits", type=int, default=0, help="override the split-K factor of the gemm-decode-* cases")
    ap.add_argument("--kv-splits", type=int, default=0, help="split-KV factor of attn-decode (0 = heuristic)")
    ap.add_argument("--tokens", type=int, default=0, help="override the token count of the gemm-decode-* cases")
    ap.add_argument("--impl", default="splitk", choices=["fixup", "cluster", "splitk"],
                    help="gemm-decode-*: fixup / cluster = split-K summed inside the kernel (last-arriver fix-up / "
                         "CTA clusters), splitk = fp32 partials left to the next kernel")
    ap.add_argument("--batch", type=int, default=0, help="attn-prefill: sequences (default 8)")
    ap.add_argument("--seq", type=int, default=0, help="attn-prefill: tokens per sequence, a multiple of 32 (default 2048)")
    ap.add_argument("--tp", type=int, default=1, help="gemm-decode-*: per-rank shard of an N-way tensor-parallel layer")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("microbench needs a GPU", file=sys.stderr)
        return 2
    pk = peaks()
    names = sorted(c for c in CASES if c != "gemm-decode-sweep") if args.case == "all" else [args.case]
    for nm in names:
        torch.manual_seed(0)
        r = CASES[nm](args)
        tbs = r["bytes"] / r["us"] / 1e6
        tfl = r["flops"] / r["us"] / 1e6
        r.update(us=round(r["us"], 2), tb_per_s=round(tbs, 3), tflops=round(tfl, 1),
                 frac_hbm=round(tbs * 1e3 / pk["hbm_gbs"], 3), frac_bf16=round(tfl / pk["bf16_tflops"], 3),
                 peaks=pk["source"])
        print(json.dumps(r), flush=True)
        torch.cuda.empty_cache()
    return 0


if __name__ == "__main__":
    sys.exit(main())
