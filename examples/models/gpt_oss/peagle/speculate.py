"""P-EAGLE speculative decoding for the gpt-oss example
(reference: examples/models/gpt_oss/peagle/speculate.py:236-459).

    python examples/models/gpt_oss/peagle/speculate.py -n 64 -k 3 --layers 6 --batch 2

Prints time to first token, verify steps, mean acceptance length and decode tokens/s, then the same
prompts through plain decoding for comparison.  With random drafter weights (no `--draft-checkpoint`)
the acceptance length is 1: the output is still identical to plain greedy decoding, each step just
emits only the target's own token.
"""
import argparse
import os
import sys
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "..", ".."))

import importlib.util  # noqa: E402


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


get_config = _load("gpt_oss_config", os.path.join(HERE, "..", "config.py")).get_config
peagle_config = _load("peagle_config", os.path.join(HERE, "config.py"))

from nkipy_b200.models.engine import GenerationEngine  # noqa: E402
from nkipy_b200.models.runner import add_common_args, build_model, build_prompts, load_tokenizer  # noqa: E402
from nkipy_b200.models.speculative import DrafterLM, SpeculativeEngine, random_drafter_weights  # noqa: E402
from nkipy_b200.models.weights import load_shard  # noqa: E402
from nkipy_b200.parallel.comm import TPGroup  # noqa: E402


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_common_args(ap)
    ap.add_argument("-k", "--num-draft-tokens", type=int, default=3)
    ap.add_argument("--draft-checkpoint", default=None, help="directory with the prepared drafter shard")
    args = ap.parse_args()
    tp = TPGroup.from_env()
    cfg = get_config(args.model)
    target = build_model(cfg, args, tp)
    cfg = target.cfg
    ecfg = peagle_config.get_eagle_config(cfg, args.num_draft_tokens)
    if args.tiny:
        ecfg.intermediate_size, ecfg.draft_vocab_size = 512, min(ecfg.draft_vocab_size, cfg.vocab_size)
    dw = (load_shard(args.draft_checkpoint, 0, device=tp.device) if args.draft_checkpoint
          else random_drafter_weights(ecfg, device=tp.device, seed=args.seed + 1))
    drafter = DrafterLM(ecfg, dw, tp.device)
    prompts = build_prompts(args, cfg, load_tokenizer(args.model))
    max_len = max(len(p) for p in prompts) + args.max_new_tokens + 64
    spec = SpeculativeEngine(target, drafter, max_batch=len(prompts), max_seq_len=max_len)
    spec.generate([p[:16] for p in prompts], 4)                    # warm-up
    spec.stats.__init__()
    out = spec.generate(prompts, args.max_new_tokens)
    s = spec.stats
    n = sum(len(o) for o in out)
    print(f"Time to first token: {s.ttft_s:.3f}s")
    print(f"Generated {n} tokens in {s.steps // len(prompts)} verify steps")
    print(f"Mean acceptance length: {s.mean_acceptance:.2f} (K={spec.K})")
    print(f"Decode tokens/sec: {n / max(s.decode_s, 1e-9):.2f}  (draft {s.draft_s:.3f}s, verify {s.verify_s:.3f}s)")
    eng = GenerationEngine(target, max_batch=len(prompts), max_seq_len=max_len,
                           use_cuda_graph=tp.device.type == "cuda" and not args.no_graph)
    eng.generate([p[:16] for p in prompts], 4)
    eng.stats.__init__()
    t0 = time.perf_counter()
    base = eng.generate(prompts, args.max_new_tokens)
    print(f"Base decode tokens/sec: {eng.stats.summary()['decode_tokens_per_s']:.2f} "
          f"({time.perf_counter() - t0:.3f}s wall)")
    same = sum(a == b for o, r in zip(out, base) for a, b in zip(o, r)) / max(1, n)
    print(f"Token agreement with plain decoding: {same:.3f}")


if __name__ == "__main__":
    main()
