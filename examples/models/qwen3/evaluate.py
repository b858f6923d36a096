"""Accuracy and latency evaluation of the serving path against the plain PyTorch implementation of the
same model and weights (the reference compares with the Hugging Face model and prints the same kind of
report, examples/models/qwen3/evaluate.py:117-368).

For a few prompts it reports the fraction of greedy tokens on which the two implementations agree, the
largest gap between the chosen token's fp32-oracle logit and the best logit (in units of the logit
standard deviation), time to first token and decode tokens/s of both paths.

    python examples/models/qwen3/evaluate.py --layers 4 --batch 4 --prompt-len 64 -n 16
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", ".."))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from config import get_config  # noqa: E402

from nkipy_b200.models.engine import GenerationEngine  # noqa: E402
from nkipy_b200.models.reference import EagerTransformer  # noqa: E402
from nkipy_b200.models.runner import add_common_args, build_prompts, load_tokenizer  # noqa: E402
from nkipy_b200.models.transformer import TransformerLM  # noqa: E402
from nkipy_b200.models.weights import load_shard, random_weights  # noqa: E402
from nkipy_b200.parallel.comm import TPGroup  # noqa: E402


def evaluate(cfg, args):
    tp = TPGroup.from_env()
    dev = tp.device
    weights = (load_shard(args.checkpoint, tp.rank, device=dev) if args.checkpoint
               else random_weights(cfg, tp.rank, tp.world_size, device=dev, seed=args.seed, std=0.05))
    model = TransformerLM(cfg, weights, tp, device=dev)
    prompts = build_prompts(args, cfg, load_tokenizer(args.model))
    n = args.max_new_tokens
    eng = GenerationEngine(model, max_batch=len(prompts), max_seq_len=len(prompts[0]) + n + 64,
                           use_cuda_graph=dev.type == "cuda" and not args.no_graph)
    eng.generate([p[:8] for p in prompts], 2)
    eng.stats.__init__()
    t0 = time.perf_counter()
    ours = eng.generate(prompts, n)
    t_ours = time.perf_counter() - t0
    ref = EagerTransformer(cfg, weights, tp, device=dev, dtype=torch.bfloat16)
    t0 = time.perf_counter()
    theirs = ref.generate(torch.tensor(prompts, device=dev), n).cpu().tolist()
    t_ref = time.perf_counter() - t0
    agree = sum(a == b for o, r in zip(ours, theirs) for a, b in zip(o, r)) / (len(prompts) * n)
    # oracle margin of our tokens (fp32 eager on the same weights), first sequence only
    oracle = EagerTransformer(cfg, weights, tp, device=dev, dtype=torch.float32)
    seq, worst = list(prompts[0]), 0.0
    for tok in ours[0]:
        oracle.reset()
        h = oracle.forward(torch.tensor([seq], device=dev))[:, -1]
        logits = (h @ oracle.w["lm_head_weight"]).float()[0]
        worst = max(worst, float((logits.max() - logits[tok]) / logits.std()))
        seq.append(tok)
    s = eng.stats.summary()
    report = {"model": cfg.name, "layers": cfg.num_layers, "batch": len(prompts), "prompt_len": len(prompts[0]),
              "new_tokens": n, "token_agreement_with_eager_bf16": round(agree, 4),
              "worst_oracle_margin_sigma": round(worst, 4), "ttft_p50_s": round(s["ttft_p50_s"], 4),
              "decode_tokens_per_s": round(s["decode_tokens_per_s"], 1), "wall_s": round(t_ours, 3),
              "eager_wall_s": round(t_ref, 3)}
    if tp.rank == 0:
        print(json.dumps(report))
    return report


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_common_args(ap)
    args = ap.parse_args()
    cfg = get_config(args.model)
    if args.layers:
        cfg.num_layers = args.layers
    evaluate(cfg, args)


if __name__ == "__main__":
    main()
