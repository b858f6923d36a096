"""Per-kernel time breakdown of one decode step.

    python -m nkipy_b200.models.breakdown --model llama3-8b [--shard-of 8] [--layers 4]
    python -m torch.distributed.run --nproc-per-node 8 ... -m nkipy_b200.models.breakdown --model llama3-8b

Every entry point of the kernel library that a decode step calls is wrapped with a
pair of CUDA events on the launching stream; the step is run eagerly (no graph), so
each pair brackets exactly one library call (one or two kernels) and the gaps the
host leaves between launches are not counted.  The table gives, per distinct call
(name + shape), launches per step, the mean device time of one call (max over
ranks) and its share; the last lines compare the sum of the isolated calls with the
time of the same step replayed from a CUDA graph, where programmatic dependent
launch overlaps neighbouring kernels.

``--shard-of N`` runs the per-rank shard of an N-way tensor-parallel model on this one
GPU with the fused push / reduce kernels looping back to the same GPU: it shows the
kernel-side floor of an N-GPU step without any NVLink traffic.

The reference reports only whole-step timers (examples/models/gpt_oss/peagle/speculate.py:351-373).
"""

from __future__ import annotations

import argparse
import collections
import json
import sys

import torch


class _TimedFn:
    """One library entry point with an event pair around each call.  Signature declarations
    (``restype`` / ``argtypes``) made on this object go to the real ctypes function."""

    def __init__(self, owner, name, fn):
        object.__setattr__(self, "_owner", owner)
        object.__setattr__(self, "_name", name)
        object.__setattr__(self, "_fn", fn)

    def __setattr__(self, key, value):
        setattr(self._fn, key, value)

    def __getattr__(self, key):
        return getattr(self._fn, key)

    def __call__(self, *args):
        owner = self._owner
        if not owner.enabled:
            return self._fn(*args)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = self._fn(*args)
        e1.record()
        ints = [a for a in args if isinstance(a, int) and not isinstance(a, bool) and 0 < a < (1 << 20)]
        owner.records.append((self._name, tuple(ints[:4]), e0, e1))
        return rc


class _TimedLib:
    """Proxy of the ctypes library object that brackets every ``nkb_*`` launch with events."""

    _LAUNCHERS = ("nkb_gemm", "nkb_tp_", "nkb_moe", "nkb_argmax", "nkb_rmsnorm", "nkb_add_rmsnorm", "nkb_silu",
                  "nkb_embedding", "nkb_rope", "nkb_decode_advance", "nkb_sample", "nkb_router", "nkb_paged_attn_decode",
                  "nkb_flash", "nkb_ag_gemm", "nkb_decode_gemm", "nkb_lmhead")

    def __init__(self, real):
        object.__setattr__(self, "_real", real)
        object.__setattr__(self, "records", [])
        object.__setattr__(self, "enabled", False)

    def __getattr__(self, name):
        fn = getattr(self._real, name)
        if not name.startswith(self._LAUNCHERS) or name.endswith(("_splits", "_floats")):
            return fn
        return _TimedFn(self, name, fn)

    def __setattr__(self, name, value):
        if name in ("records", "enabled"):
            object.__setattr__(self, name, value)
        else:
            setattr(self._real, name, value)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "qwen3-30b-a3b"])
    ap.add_argument("--shard-of", type=int, default=1, help="run the per-rank shard of an N-way TP model on one GPU")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)

    from .. import ops
    from ..ops import _lib
    from ..parallel.comm import TPGroup
    from . import config as C
    from .engine import GenerationEngine
    from .transformer import TransformerLM
    from .weights import random_weights

    tp = TPGroup.from_env()
    dev = tp.device
    _lib.ensure_init()
    proxy = _TimedLib(_lib.lib())
    _lib._lib = proxy

    cfg = C.llama3_8b() if args.model == "llama3-8b" else C.qwen3_30b_a3b()
    batch = args.batch or (64 if args.model == "llama3-8b" else 128)
    prompt_len = args.prompt_len or (1024 if args.model == "llama3-8b" else 512)
    if args.layers:
        cfg = cfg.scaled(num_layers=args.layers)
    n = args.shard_of
    if n > 1:
        if tp.world_size != 1:
            raise SystemExit("--shard-of is a single-GPU mode")
        cfg = cfg.shard_shapes(n)
    torch.manual_seed(0)
    weights = random_weights(cfg, tp.rank, tp.world_size, device=dev, seed=0, std=0.02)
    model = TransformerLM(cfg, weights, tp, device=dev, force_fused=n > 1)
    del weights
    eng = GenerationEngine(model, max_batch=batch, max_seq_len=prompt_len + 64 + 8 * args.steps,
                           use_cuda_graph=False)
    g = torch.Generator().manual_seed(0)
    seqs = eng.add_requests(torch.randint(0, cfg.vocab_size, (batch, prompt_len), generator=g).tolist())
    eng.prefill(seqs)
    eng.prepare_decode(32 + 8 * args.steps)
    for _ in range(3):
        eng.decode_step_device()
    eng.advance_host_state(3)
    torch.cuda.synchronize()
    tp.barrier()
    proxy.enabled = True
    per_step = []
    for _ in range(args.steps):
        proxy.records = []
        eng.decode_step_device()
        torch.cuda.synchronize()
        per_step.append(proxy.records)
    proxy.enabled = False
    eng.advance_host_state(args.steps)
    ops.raise_on_device_error()

    agg = collections.OrderedDict()
    for recs in per_step:
        for name, shape, e0, e1 in recs:
            key = (name, shape)
            a = agg.setdefault(key, [0, 0.0])
            a[0] += 1
            a[1] += e0.elapsed_time(e1) * 1e3
    keys = list(agg.keys())
    means = torch.tensor([agg[k][1] / agg[k][0] for k in keys], dtype=torch.float64, device=dev)
    if tp.world_size > 1:
        import torch.distributed as dist

        dist.all_reduce(means, op=dist.ReduceOp.MAX, group=tp.group)
    counts = [agg[k][0] // args.steps for k in keys]
    total_us = sum(float(m) * c for m, c in zip(means, counts))

    # the same step replayed from a CUDA graph
    eng.use_cuda_graph = True
    eng._ensure_graph()
    for _ in range(3):
        eng.decode_step_device()
    torch.cuda.synchronize()
    tp.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        eng.decode_step_device()
    e1.record()
    torch.cuda.synchronize()
    graph_us = tp.max_over_ranks(e0.elapsed_time(e1) * 100.0)
    ops.raise_on_device_error()

    if tp.rank == 0:
        rows = [{"call": k[0], "shape": list(k[1]), "per_step": c, "mean_us": round(float(m), 2),
                 "share": round(float(m) * c / total_us, 4)} for k, c, m in zip(keys, counts, means)]
        summary = {"model": cfg.name, "n_gpus": tp.world_size, "shard_of": n, "layers": cfg.num_layers, "batch": batch,
                   "prompt_len": prompt_len, "launch_calls_per_step": sum(counts),
                   "sum_isolated_us": round(total_us, 1), "graph_step_us": round(graph_us, 1),
                   "launches_per_step_graph": getattr(eng, "launches_per_step", None)}
        if args.json:
            print(json.dumps({"summary": summary, "rows": rows}))
        else:
            print("| call | first int args | per step | mean us (max over ranks) | share |")
            print("|---|---|---|---|---|")
            for r in rows:
                print(f"| {r['call']} | {r['shape']} | {r['per_step']} | {r['mean_us']} | {100 * r['share']:.1f} % |")
            print()
            print(json.dumps(summary))
    tp.barrier()
    if tp.world_size > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
