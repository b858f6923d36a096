#!/usr/bin/env python
"""Headline benchmark: greedy decode throughput of a Llama-3-8B-shaped model served
with tensor parallelism over N GPUs of one node (batch 64, 1024-token prompts).

    python bench.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 64 --warmup 8

A "step" is one decode step of the whole batch (one new token per sequence).  The
device-timed value replays the captured decode graph K times between CUDA events
(max over ranks); the end-to-end value drives the public ``GenerationEngine.step``
API with a pinned-host -> device copy of the token ids and a device -> host read of
the new ids every step.  Weights are random-init bf16, prompts are uniform random
token ids (seed 0); the per-step working set (weights + KV cache) is far larger than
L2, so no explicit L2 flush is needed between iterations.

``--impl reference`` reports why the reference cannot run on this hardware;
``--impl eager`` times the plain PyTorch (cuBLAS + NCCL) implementation of the same
model as the baseline arm.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

REFERENCE_UNAVAILABLE = (
    "reference (aws-neuron/nkipy) cannot be installed or run here: offline pip install fails "
    "(workspace root has no installable package; the nkipy member needs grpc_tools.protoc) and every "
    "module imports neuronxcc / needs libnrt and Trainium hardware"
)


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "eager", "eager-graph"],
                    help="eager-graph: the eager PyTorch decode step captured in a CUDA graph (static cache, position "
                         "on the device), so the comparison is not against Python launch overhead; dense models")
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "qwen3-30b-a3b", "gpt-oss-20b"])
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (result marked invalid)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--baseline-steps", type=int, default=4,
                    help="decode steps of the eager PyTorch baseline run before ours for vs_baseline (0 = skip)")
    ap.add_argument("--no-qwen3", action="store_true", help="skip the Qwen3-30B-A3B half of the headline metric")
    ap.add_argument("--qwen3-steps", type=int, default=20, help="timed decode steps of the Qwen3 half (at most --steps)")
    return ap.parse_args()


def measure_ours(args, cfg, batch, prompt_len, tp, K, W, parallelism, weights=None):
    """Build the engine for `cfg`, prefill, then time K decode steps on the device and K through the public
    host API.  Returns the fields of the result line that belong to this model."""
    import torch

    from nkipy_b200 import ops
    from nkipy_b200.models.engine import GenerationEngine, percentile
    from nkipy_b200.models.transformer import TransformerLM
    from nkipy_b200.models.weights import random_weights

    dev, world = tp.device, tp.world_size
    EXTRA_STEPS = 400        # room for the untimed steps that keep the clock sampler fed on short runs
    total_new = 2 * (K + W) + 4 + EXTRA_STEPS
    max_seq = prompt_len + total_new + 32
    t_build = time.perf_counter()
    if weights is None:
        torch.manual_seed(0)
        weights = random_weights(cfg, tp.rank, world, device=dev, seed=0, std=0.02)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (batch, prompt_len), generator=g)
    model = TransformerLM(cfg, weights, tp, device=dev)
    del weights
    torch.cuda.empty_cache()
    engine = GenerationEngine(model, max_batch=batch, max_seq_len=max_seq, use_cuda_graph=not args.no_graph,
                              enable_prefix_sharing=True)
    build_s = time.perf_counter() - t_build

    # one untimed warm-up prefill of the same shape with other tokens (module loading, first-use buffer
    # set-up of the fused collectives), as the reference does before it reports time to first token
    # (examples/models/gpt_oss/peagle/README.md:63-66); its sequences are released again
    gw = torch.Generator().manual_seed(12345)
    warm = engine.add_requests(torch.randint(0, cfg.vocab_size, (batch, prompt_len), generator=gw).tolist())
    engine.prefill(warm)
    torch.cuda.synchronize()
    engine.release(warm)
    engine.stats.__init__()
    seqs = engine.add_requests(prompts.tolist())
    tp.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    engine.prefill(seqs)
    torch.cuda.synchronize()
    prefill_s = tp.max_over_ranks(time.perf_counter() - t0)
    ttft_p50 = tp.max_over_ranks(percentile(engine.stats.ttft_s, 50))
    ops.raise_on_device_error()

    engine.prepare_decode(total_new)
    launches_per_step = getattr(engine, "launches_per_step", None)

    # ---------------- device-timed region: K graph replays, ids stay on the device
    for _ in range(W):
        engine.decode_step_device()
    engine.advance_host_state(W)
    sampler = ClockSampler(dev.index or 0)
    tp.barrier()
    torch.cuda.synchronize()
    sampler.start()
    t_sampler = time.perf_counter()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(K):
        engine.decode_step_device()
    end.record()
    torch.cuda.synchronize()
    tp.barrier()
    engine.advance_host_state(K)
    dev_ms = tp.max_over_ranks(start.elapsed_time(end))
    ops.raise_on_device_error()

    # ---------------- end-to-end region: public step() API with H2D ids + D2H ids every step
    host_ids = engine.ids_host
    host_ids.copy_(engine.ids.cpu())
    for _ in range(W):
        host_ids.copy_(engine.step(host_ids))
    engine.advance_host_state(W)
    tp.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(K):
        host_ids.copy_(engine.step(host_ids))
    torch.cuda.synchronize()
    e2e_s = tp.max_over_ranks(time.perf_counter() - t0)
    tp.barrier()
    engine.advance_host_state(K)
    ops.raise_on_device_error()
    # The sampler has been running since just before the device-timed region.  nvidia-smi needs a few
    # hundred milliseconds to deliver its first line, so a short run is followed by identical untimed
    # decode steps until the sampler has seen at least a second of this load.
    extra = 0
    while time.perf_counter() - t_sampler < 1.2 and extra < EXTRA_STEPS:
        engine.decode_step_device()
        extra += 1
        if extra % 8 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    if extra:
        engine.advance_host_state(extra)
    tp.barrier()
    clocks = sampler.stop()
    clocks["window"] = "device-timed + end-to-end regions" + (f" + {extra} identical untimed steps" if extra else "")
    out = {
        "value": batch * K / (dev_ms / 1e3), "ms_per_step": dev_ms / K, "e2e_value": batch * K / e2e_s,
        "e2e_ms_per_step": e2e_s * 1e3 / K, "ttft_p50_s": ttft_p50, "prefill_s": prefill_s,
        "launches_per_step": launches_per_step, "clocks": clocks, "build_s": build_s,
    }
    # release everything this model holds before the next one is built
    torch.cuda.synchronize()
    model.close()
    fused = getattr(tp, "fused", None)
    if fused is not None:
        fused.close()
        tp.fused = None
    del engine, model
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    return out


def measure_eager(cfg, weights, prompts, tp, steps, warmup):
    """A few decode steps of the plain PyTorch (cuBLAS + NCCL) implementation of the same model on the same
    weights: the baseline that `vs_baseline` refers to (the reference itself cannot run on this hardware).
    Returns decode tokens/s (device-timed, max over ranks)."""
    import torch

    from nkipy_b200.models.reference import EagerTransformer

    dev = tp.device
    model = EagerTransformer(cfg, weights, tp, device=dev, dtype=torch.bfloat16)
    batch, prompt_len = prompts.shape
    ids = prompts.to(dev)
    model.alloc_static_cache(batch, prompt_len + warmup + steps + 8)
    chunk = max(1, 16384 // prompt_len)
    firsts = []
    for b0 in range(0, batch, chunk):
        hh = EagerSlice(model, b0, min(batch, b0 + chunk)).forward(ids[b0:b0 + chunk], 0)
        firsts.append(model.greedy(hh[:, -1]))
    nxt = torch.cat(firsts)
    pos = prompt_len
    for _ in range(warmup):
        nxt = model.greedy(model.forward_sdpa(nxt[:, None], pos)[:, -1])
        pos += 1
    tp.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        nxt = model.greedy(model.forward_sdpa(nxt[:, None], pos)[:, -1])
        pos += 1
    end.record()
    torch.cuda.synchronize()
    ms = tp.max_over_ranks(start.elapsed_time(end))
    del model
    torch.cuda.empty_cache()
    return batch * steps / (ms / 1e3)


def main():
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    import torch

    from nkipy_b200.models import config as C
    from nkipy_b200.models.weights import random_weights
    from nkipy_b200.parallel.comm import TPGroup

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    tp = TPGroup.from_env()
    dev = tp.device
    if dev.type != "cuda":
        raise SystemExit("bench.py needs a CUDA device")
    rank0 = tp.rank == 0

    def shape_of(model_name):
        if model_name == "llama3-8b":
            return C.llama3_8b(), args.batch or 64, args.prompt_len or 1024, f"tp{world}"
        if model_name == "qwen3-30b-a3b":
            return C.qwen3_30b_a3b(), args.batch or 128, args.prompt_len or 512, f"tp{world}-ep{world}"
        # the only configuration the reference publishes numbers for: gpt-oss-20b, batch 1, greedy
        # (examples/models/gpt_oss/peagle/README.md:101-102: 31.5 / 34.7 tok/s base decode on trn2 at TP = 4)
        return C.gpt_oss_20b(), args.batch or 1, args.prompt_len or 128, f"tp{world}-ep{world}"

    cfg, batch, prompt_len, parallelism = shape_of(args.model)
    debug = False
    if args.layers:
        cfg = cfg.scaled(num_layers=args.layers)
        debug = True
    K, W = args.steps, max(args.warmup, 3)

    torch.manual_seed(0)
    weights = random_weights(cfg, tp.rank, world, device=dev, seed=0, std=0.02)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (batch, prompt_len), generator=g)

    if args.impl in ("eager", "eager-graph"):
        return run_eager(args, cfg, weights, prompts, tp, K, W, parallelism, graph=args.impl == "eager-graph")

    # baseline of the same model on the same weights, a few steps (eager PyTorch: cuBLAS, SDPA, NCCL)
    eager_value = None
    if args.baseline_steps > 0:
        eager_value = measure_eager(cfg, weights, prompts, tp, args.baseline_steps, 2)

    r = measure_ours(args, cfg, batch, prompt_len, tp, K, W, parallelism, weights=weights)
    del weights
    value = r["value"]
    published = round(value / 34.7, 2) if (args.model == "gpt-oss-20b" and batch == 1) else None
    result = {
        "metric": {"llama3-8b": "decode tokens/s (Llama-3-8B-shaped, TP over N GPUs, batch 64, prompt 1024, greedy)",
                   "qwen3-30b-a3b": "decode tokens/s (Qwen3-30B-A3B-shaped MoE, batch 128, prompt 512, greedy)",
                   "gpt-oss-20b": "decode tokens/s (gpt-oss-20b-shaped MoE, batch 1, greedy)"}[args.model],
        "value": round(value, 2),
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": K,
        "warmup": W,
        "ms_per_step": round(r["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "strong",
        # The reference publishes a number only for gpt-oss-20b at batch 1 (34.7 tok/s, best base decode on trn2);
        # for the other models the baseline is the eager PyTorch implementation measured a moment ago in this
        # process on the same weights (see "baseline").
        "vs_baseline": published if published is not None else (round(value / eager_value, 2) if eager_value else None),
        "baseline": ({"impl": "reference, published (trn2, TP=4)", "value": 34.7} if published is not None else
                     ({"impl": "eager-pytorch (cuBLAS + SDPA + NCCL), same process, same weights",
                       "value": round(eager_value, 2), "unit": "tokens/s", "steps": args.baseline_steps}
                      if eager_value else None)),
        "dtype": "bf16",
        "data": "synthetic (uniform random token ids seed 0; random-init weights N(0, 0.02))",
        "impl": "ours",
        "config": {
            "model": cfg.name, "global_batch": batch, "seq_len": prompt_len, "parallelism": parallelism,
            "layers": cfg.num_layers, "new_tokens_timed": K, "kv_cache": "paged, block 32, prefix sharing on",
            "l2": "per-step working set (weights + KV) exceeds L2; no flush", "cuda_graph": not args.no_graph,
        },
        "ttft_p50_s": round(r["ttft_p50_s"], 4),
        "prefill_s": round(r["prefill_s"], 4),
        "prefill_tokens_per_s": round(batch * prompt_len / r["prefill_s"], 1),
        "e2e": {"value": round(r["e2e_value"], 2), "unit": "tokens/s", "h2d_bytes_per_step": batch * 4,
                "d2h_bytes_per_step": batch * 4, "ms_per_step": round(r["e2e_ms_per_step"], 4)},
        "gpu_launches": (r["launches_per_step"] or 0) * K,
        "launches_per_step": r["launches_per_step"],
        "clocks": r["clocks"],
        "build_s": round(r["build_s"], 1),
    }
    # The second half of the headline metric: the Qwen3-30B-A3B-shaped MoE model (expert parallel over the same
    # GPUs), measured after the first model's memory has been released.
    if args.model == "llama3-8b" and not args.no_qwen3 and not debug:
        qcfg, qbatch, qprompt, qpar = shape_of("qwen3-30b-a3b")
        qK = max(3, min(K, args.qwen3_steps))
        q = measure_ours(args, qcfg, qbatch, qprompt, tp, qK, W, qpar)
        result.update({
            "qwen3_decode_tokens_per_s": round(q["value"], 2), "qwen3_ms_per_step": round(q["ms_per_step"], 4),
            "qwen3_ttft_p50_s": round(q["ttft_p50_s"], 4), "qwen3_prefill_s": round(q["prefill_s"], 4),
            "qwen3_e2e_tokens_per_s": round(q["e2e_value"], 2), "qwen3_launches_per_step": q["launches_per_step"],
            "qwen3_config": {"model": qcfg.name, "global_batch": qbatch, "seq_len": qprompt, "parallelism": qpar,
                             "steps": qK},
        })
    if debug:
        result["invalid"] = "debug run with a reduced layer count"
    if rank0:
        print(json.dumps(result), flush=True)
    tp.barrier()
    return 0


class EagerSlice:
    """Runs the eager model on sequences [b0, b1) of its static cache (chunked prefill)."""

    def __init__(self, model, b0, b1):
        self.model, self.b0, self.b1 = model, b0, b1

    def forward(self, ids, start_pos):
        m = self.model
        full_k, full_v = m.k_static, m.v_static
        m.k_static = [t[self.b0:self.b1] for t in full_k]
        m.v_static = [t[self.b0:self.b1] for t in full_v]
        try:
            return m.forward_sdpa(ids, start_pos)
        finally:
            m.k_static, m.v_static = full_k, full_v


def run_eager(args, cfg, weights, prompts, tp, K, W, parallelism, graph=False):
    """Baseline arm: plain PyTorch (cuBLAS, NCCL) decoder with a dense cache; with graph=True the decode step is
    captured in a CUDA graph and replayed."""
    import torch

    from nkipy_b200.models.reference import EagerTransformer

    dev = tp.device
    model = EagerTransformer(cfg, weights, tp, device=dev, dtype=torch.bfloat16)
    batch, prompt_len = prompts.shape
    ids = prompts.to(dev)
    tp.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    model.alloc_static_cache(batch, prompt_len + W + K + 12)
    chunk0 = max(1, 16384 // prompt_len)
    EagerSlice(model, 0, min(batch, chunk0)).forward(ids[:chunk0].flip(1), 0)      # untimed warm-up chunk
    torch.cuda.synchronize()
    tp.barrier()
    t0 = time.perf_counter()
    # prefill in chunks of 16 sequences like the engine does, so that TTFT p50 is comparable
    chunk = max(1, 16384 // prompt_len)
    ttfts, firsts = [], []
    for b0 in range(0, batch, chunk):
        sub = EagerSlice(model, b0, min(batch, b0 + chunk))
        hh = sub.forward(ids[b0:b0 + chunk], 0)
        firsts.append(model.greedy(hh[:, -1]))
        torch.cuda.synchronize()
        ttfts += [time.perf_counter() - t0] * (min(batch, b0 + chunk) - b0)
    nxt = torch.cat(firsts)
    prefill_s = time.perf_counter() - t0
    ttfts.sort()
    ttft_p50 = ttfts[len(ttfts) // 2]
    pos = prompt_len
    step_graph = None
    if graph:
        pos_t = torch.tensor([pos], dtype=torch.int64, device=dev)
        cur = nxt.clone()

        def body():
            h = model.forward_decode_static(cur[:, None], pos_t)
            cur.copy_(model.greedy(h[:, -1]))
            pos_t.add_(1)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        step_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(step_graph):
            body()

    def step():
        nonlocal nxt, pos
        if step_graph is not None:
            step_graph.replay()
            return
        h = model.forward_sdpa(nxt[:, None], pos)
        nxt = model.greedy(h[:, -1])
        pos += 1

    for _ in range(W):
        step()
    sampler = ClockSampler(dev.index or 0)
    tp.barrier()
    torch.cuda.synchronize()
    sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(K):
        step()
    end.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = tp.max_over_ranks(start.elapsed_time(end))
    if tp.rank == 0:
        print(json.dumps({
            "metric": "decode tokens/s", "impl": "eager-pytorch-graph" if graph else "eager-pytorch", "value": round(batch * K / (ms / 1e3), 2),
            "unit": "tokens/s", "n_gpus": tp.world_size, "steps": K, "warmup": W,
            "ms_per_step": round(ms / K, 4), "higher_is_better": True, "scaling": "strong", "dtype": "bf16",
            "data": "synthetic", "ttft_p50_s": round(ttft_p50, 4), "prefill_s": round(prefill_s, 4),
            "config": {"model": cfg.name, "global_batch": batch, "seq_len": prompt_len, "parallelism": parallelism},
            "clocks": clocks}), flush=True)
    tp.barrier()
    return 0


def _entry():
    rc = main()
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass
    return rc


if __name__ == "__main__":
    sys.exit(_entry())
