"""Command-line plumbing shared by the example entry points (examples/models/*): weights from prepared
shards or random init, prompts from a tokenizer or synthetic ids, generation through the paged engine
and the timing lines the reference scripts print (examples/models/qwen3/qwen3.py:495-537)."""

from __future__ import annotations

import argparse
import os
import time
from typing import List, Optional

import torch

from ..parallel.comm import TPGroup
from .config import ModelConfig
from .engine import GenerationEngine
from .transformer import TransformerLM
from .weights import load_shard, random_weights


def add_common_args(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("prompt", nargs="?", default=None, help="prompt text (needs --model with a tokenizer)")
    ap.add_argument("--checkpoint", default=None, help="directory with shard_{rank}.safetensors; random init if absent")
    ap.add_argument("--model", default=None, help="Hugging Face model directory (tokenizer / config)")
    ap.add_argument("-n", "--max-new-tokens", type=int, default=64)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt-len", type=int, default=128, help="synthetic prompt length when no tokenizer is given")
    ap.add_argument("--max-seq-len", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (quick runs)")
    ap.add_argument("--moe-parallel", choices=["ep", "tp"], default="ep")
    ap.add_argument("--no-graph", action="store_true", help="do not capture the decode step in a CUDA graph")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--tiny", action="store_true",
                    help="shrink the model (hidden 256, vocabulary 2048, <= 8 experts) for quick functional runs")


def load_tokenizer(path: Optional[str]):
    if not path:
        return None
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(path)


def build_prompts(args, cfg: ModelConfig, tokenizer) -> List[List[int]]:
    if tokenizer is not None and args.prompt:
        ids = tokenizer(args.prompt)["input_ids"]
        return [list(ids) for _ in range(args.batch)]
    g = torch.Generator().manual_seed(args.seed)
    return torch.randint(0, cfg.vocab_size, (args.batch, args.prompt_len), generator=g).tolist()


def shrink(cfg: ModelConfig) -> ModelConfig:
    """Same architecture features, toy sizes."""
    over = dict(vocab_size=2048, hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=512,
                max_position=min(cfg.max_position, 4096))
    if cfg.is_moe:
        over.update(num_experts=min(cfg.num_experts, 8), top_k=min(cfg.top_k, 2), moe_intermediate_size=128,
                    intermediate_size=0)
    if cfg.layer_types is not None:
        over["layer_types"] = cfg.layer_types[: max(cfg.num_layers, 1)]
    if cfg.sliding_window:
        over["sliding_window"] = min(cfg.sliding_window, 16)
    return cfg.scaled(**over)


def build_model(cfg: ModelConfig, args, tp: TPGroup) -> TransformerLM:
    if args.layers:
        cfg.num_layers = args.layers
        if cfg.layer_types is not None:
            cfg.layer_types = cfg.layer_types[: args.layers]
    if getattr(args, "tiny", False):
        cfg = shrink(cfg)
    if args.checkpoint:
        weights = load_shard(args.checkpoint, tp.rank, device=tp.device)
    else:
        weights = random_weights(cfg, tp.rank, tp.world_size, device=tp.device, seed=args.seed,
                                 moe_parallel=args.moe_parallel)
    return TransformerLM(cfg, weights, tp, device=tp.device, moe_parallel=args.moe_parallel)


def run_generation(cfg: ModelConfig, args) -> int:
    tp = TPGroup.from_env()
    tokenizer = load_tokenizer(args.model)
    model = build_model(cfg, args, tp)
    prompts = build_prompts(args, cfg, tokenizer)
    max_len = min(args.max_seq_len, max(len(p) for p in prompts) + args.max_new_tokens + 64)
    eng = GenerationEngine(model, max_batch=len(prompts), max_seq_len=max_len,
                           use_cuda_graph=not args.no_graph and tp.device.type == "cuda")
    eng.generate([p[:8] for p in prompts], 2)            # warm-up (graph capture, autotuned splits)
    eng.stats.__init__()
    tp.barrier()
    t0 = time.perf_counter()
    out = eng.generate(prompts, args.max_new_tokens)
    dt = time.perf_counter() - t0
    if tp.rank == 0:
        s = eng.stats.summary()
        print(f"Time to first token: {s.get('ttft_p50_s', 0.0):.3f}s")
        n = sum(len(o) for o in out)
        print(f"Generated {n} tokens in {dt:.3f}s")
        print(f"Decode tokens/sec: {s.get('decode_tokens_per_s', n / max(dt, 1e-9)):.2f}")
        if tokenizer is not None:
            print(tokenizer.decode(out[0]))
        else:
            print("first sequence ids:", out[0][:32])
    tp.barrier()
    if tp.world_size > 1:
        torch.distributed.destroy_process_group()
    return 0
