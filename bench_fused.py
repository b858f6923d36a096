"""Micro-benchmark of the GEMM + collective kernels against NCCL + cuBLAS.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench_fused.py

Shapes (per rank, bf16):
  rs: X[M, 8192/tp] @ W[8192/tp, 8192] -> reduce-scatter over rows       (row-parallel o_proj / down)
  ag: all-gather(X[M/tp, 8192]) @ W[8192, 28672/tp]                      (column-parallel gate_up)
  ar: X[M, 8192/tp] @ W[8192/tp, 8192] -> all-reduce + residual + RMSNorm, M <= 128 (the decode form of rs:
      weights on the 128-row MMA side, split-K, partial tiles pushed to every peer, reducing norm kernel)
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ms", type=str, default="16,64,256,1024,4096,16384")
    ap.add_argument("--ops", type=str, default="ar,rs,ag")
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
