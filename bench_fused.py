"""Micro-benchmark of the GEMM + collective kernels against NCCL + cuBLAS.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench_fused.py

Shapes (per rank, bf16):
  rs: X[M, 8192/tp] @ W[8192/tp, 8192] -> reduce-scatter over rows       (row-parallel o_proj / down)
  ag: all-gather(X[M/tp, 8192]) @ W[8192, 28672/tp]                      (column-parallel gate_up)
  ar: X[M, 8192/tp] @ W[8192/tp, 8192] -> all-reduce + residual + RMSNorm, M <= 128 (the decode form of rs:
      weights on the 128-row MMA side, split-K, partial tiles pushed to every peer, reducing norm kernel)
  moe: one Qwen3-30B-A3B-shaped expert-parallel MoE block (hidden 2048, 128 experts / tp per rank, top-8, expert
      FFN 768) on M replicated tokens, M <= 256: router, device-built dispatch, two grouped tcgen05 GEMMs, then the
      combine whose kernel stores every token's weighted partial sum into all peers' buffers (the all-to-all of
      this layout) followed by the summing residual + RMSNorm kernel.  Baseline: the same experts with a local
      combine, NCCL all-reduce and a separate residual + RMSNorm.  `combine_*` fields time the exchange alone.
      From 256 tokens per rank on the tokens are sharded over the ranks and the block runs over the token
      all-to-all in peer memory (op "moe_a2a_block"): dispatch, arrival-gated grouped GEMMs, combine;
      `dispatch_frac_link` / `combine_frac_link` = bytes crossing NVLink each way / 770 GB/s / measured time.
for M = 16 ... 16384.  "fused" is one kernel per rank (csrc/kernels/gemm_comm.cu: tcgen05 tiles + peer stores
over NVLink + arrival counters); "baseline" is torch.matmul (cuBLAS) with NCCL reduce_scatter_tensor /
all_gather_into_tensor.  Every iteration is timed on the device with CUDA events after an L2 flush (a 256 MB
memset) and a barrier; the reported time is the median over iterations of the max over ranks.  The roofline is
the slowest of FLOPs / measured cuBLAS bf16 throughput, bytes leaving this GPU / 770 GB/s (measured peer copy
per direction) and operand + result bytes / measured HBM copy bandwidth; `frac_roofline` = roofline time / achieved time.  Rank 0 prints one JSON line per (op, M).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from nkipy_b200 import ops  # noqa: E402
from nkipy_b200.ops.microbench import peaks  # noqa: E402
from nkipy_b200.parallel.comm import TPGroup  # noqa: E402
from nkipy_b200.parallel.symm import AllGatherGemm, FusedTP, GemmReduceScatter  # noqa: E402

NVLINK_GBS = 770.0


def timed(tp, fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        torch.cuda.synchronize()
        tp.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(tp.max_over_ranks(e0.elapsed_time(e1) * 1e3))
    ts.sort()
    return ts[len(ts) // 2]


def bench_moe(tp, m, args, pk, flush, g):
    from nkipy_b200.models import config as C
    from nkipy_b200.models.moe import MoEBlock

    n_r, dev = tp.world_size, tp.device
    cfg = C.qwen3_30b_a3b()
    H, E, I, K = cfg.hidden_size, cfg.num_experts, cfg.moe_intermediate_size, cfg.top_k
    e_l = E // n_r

    class LW:
        pass

    lw = LW()
    gs = torch.Generator(device=dev).manual_seed(3)          # replicated tensors: same seed on every rank
    lw.router = (torch.randn(E, H, device=dev, generator=gs) * 0.02).to(torch.bfloat16)
    lw.router_bias = lw.gate_up_bias = lw.down_bias = None
    lw.gate_up = (torch.randn(e_l, 2 * I, H, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    lw.down = (torch.randn(e_l, H, I, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(m, H, device=dev, generator=gs).to(torch.bfloat16)
    resid = torch.randn(m, H, device=dev, generator=gs).to(torch.bfloat16)
    wn = torch.ones(H, device=dev, dtype=torch.bfloat16)
    blk = MoEBlock(cfg, tp, "ep")
    fused = FusedTP(tp, m, H) if n_r > 1 else None
    state = {"i": 0}

    def tick():
        if state["i"] % 2 == 0:
            fused.begin_step()
        state["i"] += 1

    def run():
        if fused is None:
            return base()
        tick()
        y_sorted, plan, weights = blk._experts(lw, x)
        return fused.moe_combine_allreduce_add_rmsnorm(y_sorted, plan.pair_pos, weights, m, resid, wn, cfg.rms_eps)[1]

    def base():
        y = blk.forward(lw, x)                               # local combine + NCCL all-reduce
        return ops.add_rmsnorm(y, wn, residual_in=resid, eps=cfg.rms_eps)[1]

    y_sorted, plan, weights = blk._experts(lw, x)

    def run_c():
        if fused is None:
            return base_c()
        tick()
        return fused.moe_combine_allreduce_add_rmsnorm(y_sorted, plan.pair_pos, weights, m, resid, wn, cfg.rms_eps)[1]

    def base_c():
        y = ops.moe_combine(y_sorted, plan.pair_pos, weights, m)
        tp.all_reduce(y)
        return ops.add_rmsnorm(y, wn, residual_in=resid, eps=cfg.rms_eps)[1]

    a, b = run().float(), base().float()
    if fused is not None:
        run()
    rel = ((a - b).norm() / b.norm().clamp_min(1e-6)).item()
    even = args.iters + (args.iters + args.warmup) % 2
    t_f, t_b = timed(tp, run, even, args.warmup, flush), timed(tp, base, args.iters, args.warmup, flush)
    t_fc, t_bc = timed(tp, run_c, even, args.warmup, flush), timed(tp, base_c, args.iters, args.warmup, flush)
    pairs_local = m * K / n_r
    active = e_l * (1.0 - (1.0 - 1.0 / E) ** (m * K))        # expected number of local experts with a token
    t_h = (active * 3 * H * I + E * H) * 2 / (pk["hbm_gbs"] * 1e3)
    t_c = 2.0 * pairs_local * 3 * H * I / (pk["bf16_tflops"] * 1e6)
    link_bytes = (n_r - 1) * m * H * 2                       # every rank's partial rows go to every peer
    t_l = link_bytes / (NVLINK_GBS * 1e3)
    roof = max(t_h, t_c, t_l)
    status = ops.device_status()
    if tp.rank == 0:
        print(json.dumps({
            "op": "moe_ep_block", "tp": n_r, "m": m, "experts_per_rank": e_l, "fused_us": round(t_f, 1),
            "nccl_us": round(t_b, 1), "speedup": round(t_b / t_f, 2), "roofline_us": round(roof, 1),
            "frac_roofline": round(roof / t_f, 3), "bound": "hbm" if roof == t_h else ("nvlink" if roof == t_l else "compute"),
            "combine_fused_us": round(t_fc, 1), "combine_nccl_us": round(t_bc, 1),
            "combine_link_us": round(t_l, 2), "combine_frac_link": round(t_l / t_fc, 3),
            "rel_err_vs_baseline": round(rel, 5), "status": status, "peaks": pk["source"]}), flush=True)
    torch.cuda.synchronize()
    tp.barrier()
    if fused is not None:
        fused.close()


def bench_moe_a2a(tp, m, args, pk, flush, g):
    """One Qwen3-30B-A3B-shaped expert-parallel MoE block on m tokens sharded over the ranks (m / tp each):
    the token all-to-all in peer memory against replicating the tokens with NCCL (all-gather, local experts,
    reduce-scatter).  `dispatch_*` / `combine_*` time the two exchanges alone against the bytes they move."""
    from nkipy_b200.models import config as C
    from nkipy_b200.models.moe import MoEBlock
    from nkipy_b200.parallel.moe_a2a import MoEAllToAll

    n_r, dev = tp.world_size, tp.device
    cfg = C.qwen3_30b_a3b()
    H, E, I, K = cfg.hidden_size, cfg.num_experts, cfg.moe_intermediate_size, cfg.top_k
    e_l, t_l = E // n_r, m // n_r

    class LW:
        pass

    lw = LW()
    gs = torch.Generator(device=dev).manual_seed(3)          # replicated tensors: same seed on every rank
    lw.router = (torch.randn(E, H, device=dev, generator=gs) * 0.02).to(torch.bfloat16)
    lw.router_bias = lw.gate_up_bias = lw.down_bias = None
    lw.gate_up = (torch.randn(e_l, 2 * I, H, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    lw.down = (torch.randn(e_l, H, I, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(t_l, H, device=dev, generator=g).to(torch.bfloat16)      # this rank's tokens
    blk = MoEBlock(cfg, tp, "ep")
    a2a = MoEAllToAll(tp, t_l, K, H, E, capacity_factor=2.0)
    weights, experts = blk.route(lw, x)

    def run():
        return a2a.forward(x, experts, weights, lw.gate_up, lw.down)

    def base():
        full = tp.all_gather(x).reshape(m, H)
        w_all, e_all = blk.route(lw, full)
        plan = ops.moe_dispatch(full, e_all, blk.expert_lo, blk.num_local)
        h = ops.grouped_linear(plan.x_sorted, lw.gate_up, plan.offsets, max_rows_per_group=m, gated=True,
                               tiles=plan.tiles)
        y_sorted = ops.grouped_linear(h, lw.down, plan.offsets, max_rows_per_group=m, tiles=plan.tiles)
        y = ops.moe_combine(y_sorted, plan.pair_pos, w_all, m)
        return tp.reduce_scatter(y)

    a, b = run().float(), base().float()
    rel = ((a - b).norm() / b.norm().clamp_min(1e-6)).item()
    t_f, t_b = timed(tp, run, args.iters, args.warmup, flush), timed(tp, base, args.iters, args.warmup, flush)
    t_d = timed(tp, lambda: a2a.dispatch(x, experts), args.iters, args.warmup, flush)
    a2a.run_experts(lw.gate_up, lw.down)
    t_c = timed(tp, lambda: a2a.combine(weights, t_l), args.iters, args.warmup, flush)
    link_bytes = a2a.bytes_sent_per_rank(t_l)                 # each way
    t_l_us = link_bytes / (NVLINK_GBS * 1e3)
    flops = 2.0 * t_l * K * 3 * H * I                          # expected pairs per rank under uniform routing
    t_cmp = flops / (pk["bf16_tflops"] * 1e6)
    t_h = (e_l * 3 * H * I * 2 + 4 * t_l * K * H * 2) / (pk["hbm_gbs"] * 1e3)
    roof = max(t_cmp, 2 * t_l_us, t_h)
    status = ops.device_status()
    if tp.rank == 0:
        print(json.dumps({
            "op": "moe_a2a_block", "tp": n_r, "tokens": m, "tokens_per_rank": t_l, "experts_per_rank": e_l,
            "fused_us": round(t_f, 1), "nccl_us": round(t_b, 1), "speedup": round(t_b / t_f, 2),
            "roofline_us": round(roof, 1), "frac_roofline": round(roof / t_f, 3),
            "bound": "compute" if roof == t_cmp else ("nvlink" if roof == 2 * t_l_us else "hbm"),
            "dispatch_us": round(t_d, 1), "combine_us": round(t_c, 1), "link_us_each_way": round(t_l_us, 1),
            "dispatch_frac_link": round(t_l_us / t_d, 3), "combine_frac_link": round(t_l_us / t_c, 3),
            "link_mb_each_way": round(link_bytes / 1e6, 1), "rel_err_vs_baseline": round(rel, 5), "status": status,
            "peaks": pk["source"]}), flush=True)
    torch.cuda.synchronize()
    tp.barrier()
    a2a.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ms", type=str, default="16,32,64,128,256,512,1024,2048,4096,8192,16384")
    ap.add_argument("--ops", type=str, default="ar,rs,ag,moe")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--inter", type=int, default=28672)
    ap.add_argument("--comm-ctas", type=int, default=0, help="CTAs that push slabs in ag_gemm (0 = 2 per rank)")
    args = ap.parse_args()
    tp = TPGroup.from_env()
    n_r = tp.world_size
    dev = tp.device
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(11 + tp.rank)
    H, I = args.hidden, args.inter
    for op in args.ops.split(","):
        for m in [int(v) for v in args.ms.split(",")]:
            if m % n_r:
                continue
            if op == "moe":
                # few tokens: replicated-token form; from 256 tokens per rank on: the token all-to-all
                if m <= 256:
                    bench_moe(tp, m, args, pk, flush, g)
                if m // n_r >= 256:
                    bench_moe_a2a(tp, m, args, pk, flush, g)
                continue
            if op == "ar":
                if m > 128 or n_r < 2:
                    continue
                k, n = H // n_r, H
                x = torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16)
                w = (torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
                resid = torch.randn(m, n, device=dev, generator=g).to(torch.bfloat16)
                dist.broadcast(resid, 0)
                wn = torch.ones(n, device=dev, dtype=torch.bfloat16)
                fused = FusedTP(tp, m, n)
                state = {"i": 0}

                def run():
                    if state["i"] % 2 == 0:
                        fused.begin_step()
                    state["i"] += 1
                    return fused.gemm_allreduce_add_rmsnorm(x, w, resid, wn, None, 1e-5, splits=4)[1]

                def base():
                    y = torch.matmul(x, w.T)
                    dist.all_reduce(y)
                    h = (y.float() + resid.float())
                    return (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * wn.float()).to(torch.bfloat16)

                flops = 2.0 * m * k * n
                link_bytes = (n_r - 1) * m * n * 2
            elif op == "rs":
                k, n = H // n_r, H
                x = torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16)
                w = (torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
                fused = GemmReduceScatter(tp, m, n)
                out_b = torch.empty((m // n_r, n), dtype=torch.bfloat16, device=dev)

                def base():
                    y = torch.matmul(x, w.T)
                    if n_r > 1:
                        dist.reduce_scatter_tensor(out_b, y)
                    else:
                        out_b.copy_(y)

                run = lambda: fused(x, w)  # noqa: E731
                flops = 2.0 * m * k * n
                link_bytes = (n_r - 1) / n_r * m * n * 2
            else:
                k, n = H, I // n_r
                x = torch.randn(m // n_r, k, device=dev, generator=g).to(torch.bfloat16)
                w = (torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
                fused = AllGatherGemm(tp, m, k, comm_ctas=args.comm_ctas)
                xg = torch.empty((m, k), dtype=torch.bfloat16, device=dev)

                def base():
                    if n_r > 1:
                        dist.all_gather_into_tensor(xg, x)
                    else:
                        xg.copy_(x)
                    return torch.matmul(xg, w.T)

                run = lambda: fused(x, w)  # noqa: E731
                flops = 2.0 * m * k * n
                link_bytes = (n_r - 1) * (m // n_r) * k * 2
            # numerics of the fused path against the baseline on this rank
            a = run().float()
            if op == "ar":
                run()          # keep the two alternating buffers of the fused op in step
            if op == "rs":
                base()
                b = out_b.float()
            else:
                b = base().float()
            rel = ((a - b).norm() / b.norm().clamp_min(1e-6)).item()
            t_f = timed(tp, run, args.iters + (args.iters + args.warmup) % 2, args.warmup, flush)
            t_b = timed(tp, base, args.iters, args.warmup, flush)
            t_c = flops / (pk["bf16_tflops"] * 1e6)
            t_l = link_bytes / (NVLINK_GBS * 1e3)
            t_h = (x.numel() + w.numel() + m * n // (n_r if op == "rs" else 1)) * 2 / (pk["hbm_gbs"] * 1e3)
            roof = max(t_c, t_l, t_h)
            status = ops.device_status()
            if tp.rank == 0:
                print(json.dumps({
                    "op": {"rs": "gemm_rs", "ag": "ag_gemm", "ar": "gemm_ar_norm"}[op], "tp": n_r, "m": m, "n": n, "k": k,
                    "fused_us": round(t_f, 1), "nccl_cublas_us": round(t_b, 1), "speedup": round(t_b / t_f, 2),
                    "roofline_us": round(roof, 1), "frac_roofline": round(roof / t_f, 3),
                    "bound": "compute" if roof == t_c else ("nvlink" if roof == t_l else "hbm"), "tflops": round(flops / t_f / 1e6, 1), "rel_err_vs_baseline": round(rel, 5),
                    "status": status, "peaks": pk["source"]}), flush=True)
            torch.cuda.synchronize()
            tp.barrier()
            fused.close()
            del fused, x, w
    if n_r > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
