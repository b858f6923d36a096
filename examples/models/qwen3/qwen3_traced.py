"""Qwen3-MoE through the tracing frontend: every layer, the embedding and the sampler are NumPy kernel functions
(`qwen3_kernels/` plus the Llama example's attention, norms and sampler).

    python examples/models/qwen3/qwen3_traced.py --layers 2 --experts 8 --top-k 2 -n 8

backend "numpy":  the kernel functions run directly on NumPy arrays (CPU direct mode);
backend "traced": each function is traced once per shape into the IR and the graphs are evaluated by the
                  interpreter, which is what the compiler and the device runtime start from.
The serving path of this model on the GPU is `qwen3.py` next to this file (hand-written kernels, expert parallelism).
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from typing import Dict, List

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(_HERE, "..", "..", ".."))
sys.path.insert(0, os.path.join(_HERE, "..", "llama"))
sys.path.insert(0, _HERE)

from llama import _np, embed  # noqa: E402
from llama_kernels import greedy_token  # noqa: E402
from qwen3_kernels import decode_layer, prefill_layer  # noqa: E402

_ORDER = ["qkv_weight", "o_weight", "q_norm", "k_norm", "router_weight", "gate_up_weight", "down_weight",
          "input_norm", "post_norm", "cache_k", "cache_v"]


class TracedQwen3:
    def __init__(self, cfg, weights: Dict, batch: int, prompt_len: int, max_seq_len: int, backend: str = "numpy"):
        if not (cfg.is_moe and cfg.qk_norm) or cfg.router_mode != "softmax_topk":
            raise ValueError("this example covers Qwen3-MoE layers (QK-norm, softmax-then-top-k routing)")
        if backend not in ("numpy", "traced"):
            raise ValueError("backends: numpy, traced")
        self.cfg, self.batch, self.prompt_len, self.max_seq_len, self.backend = cfg, batch, prompt_len, max_seq_len, backend
        d = np.float32
        self.scalars = dict(n_heads=cfg.num_heads, n_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                            rope_theta=float(cfg.rope_theta), norm_eps=float(cfg.rms_eps), top_k=cfg.top_k)
        self.host = {"table": _np(weights["tok_embedding"], d), "final_norm": _np(weights["norm_weight"], d),
                     "lm_head": _np(weights["lm_head_weight"], d)}
        self.layers: List[Dict[str, np.ndarray]] = []
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            self.layers.append({
                "qkv_weight": _np(weights[p + "qkv_weight"], d), "o_weight": _np(weights[p + "o_weight"], d),
                "q_norm": _np(weights[p + "q_norm_weight"], d), "k_norm": _np(weights[p + "k_norm_weight"], d),
                "router_weight": _np(weights[p + "router_weight"], d),
                "gate_up_weight": _np(weights[p + "gate_up_weight"], d), "down_weight": _np(weights[p + "down_weight"], d),
                "input_norm": _np(weights[p + "input_layernorm_weight"], d),
                "post_norm": _np(weights[p + "post_attention_layernorm_weight"], d),
                "cache_k": np.zeros((batch, max_seq_len, cfg.num_kv_heads, cfg.head_dim), d),
                "cache_v": np.zeros((batch, max_seq_len, cfg.num_kv_heads, cfg.head_dim), d)})
        self.graphs = {}

    # ------------------------------------------------------------------ one layer
    def _graph(self, name, fn, example_args, scalars):
        from nkipy_b200.core.compile import trace

        if name not in self.graphs:
            self.graphs[name] = trace(fn).specialize(*[a.copy() for a in example_args], **scalars)
        return self.graphs[name]

    def _layer(self, which: str, x, lw, start_pos=None):
        args = [lw[k] for k in _ORDER]
        lead = [x] if start_pos is None else [x, start_pos]
        fn = prefill_layer if which == "prefill" else decode_layer
        if self.backend == "numpy":
            return fn(*lead, *args, **self.scalars)               # writes the caches in place
        from nkipy_b200.core.interp import evaluate

        g = self._graph(which, fn, lead + args, self.scalars)
        out = evaluate(g, lead + args)
        names = [o.name for o in g.outputs]
        lw["cache_k"], lw["cache_v"] = np.asarray(out[names.index("cache_k")]), np.asarray(out[names.index("cache_v")])
        return np.asarray(out[names.index("output0")])

    def _sample(self, x):
        if self.backend == "numpy":
            return greedy_token(x, self.host["final_norm"], self.host["lm_head"], self.scalars["norm_eps"])
        from nkipy_b200.core.interp import evaluate

        g = self._graph(f"sample{x.shape[1]}", greedy_token, [x, self.host["final_norm"], self.host["lm_head"]],
                        dict(norm_eps=self.scalars["norm_eps"]))
        return np.asarray(evaluate(g, [x, self.host["final_norm"], self.host["lm_head"]])[0])

    # ------------------------------------------------------------------ generation
    def generate(self, prompts, new_tokens: int) -> List[List[int]]:
        prompts = np.asarray(prompts, dtype=np.int32)
        B, T = prompts.shape
        if (B, T) != (self.batch, self.prompt_len):
            raise ValueError(f"built for prompts of shape {(self.batch, self.prompt_len)}, got {(B, T)}")
        if T + new_tokens > self.max_seq_len:
            raise ValueError("prompt + new tokens exceed the cache length")
        out = [[] for _ in range(B)]
        x = embed(prompts, self.host["table"])
        for lw in self.layers:
            x = self._layer("prefill", x, lw)
        tok = self._sample(x)
        for step in range(new_tokens):
            for b in range(B):
                out[b].append(int(tok[b]))
            if step + 1 == new_tokens:
                break
            x = embed(np.asarray(tok).reshape(B, 1).astype(np.int32), self.host["table"])
            pos = np.array([T + step], np.int32)
            for lw in self.layers:
                x = self._layer("decode", x, lw, pos)
            tok = self._sample(x)
        return out


def main(argv=None) -> int:
    import torch

    from nkipy_b200.models import config as C
    from nkipy_b200.models.weights import random_weights

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--prompt-len", type=int, default=12)
    ap.add_argument("-n", "--new-tokens", type=int, default=8)
    ap.add_argument("--backend", choices=["numpy", "traced"], default="traced")
    args = ap.parse_args(argv)
    cfg = C.tiny(hidden_size=args.hidden, head_dim=64, num_heads=args.hidden // 64, num_kv_heads=2, vocab_size=1024,
                 num_layers=args.layers, qk_norm=True, num_experts=args.experts, top_k=args.top_k,
                 moe_intermediate_size=args.hidden // 2, intermediate_size=0, rms_eps=1e-6)
    w = random_weights(cfg, seed=0, std=0.05, dtype=torch.float32)
    model = TracedQwen3(cfg, w, args.batch, args.prompt_len, args.prompt_len + args.new_tokens, backend=args.backend)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt_len), generator=g).numpy()
    t0 = time.time()
    toks = model.generate(prompts, args.new_tokens)
    print(f"backend {model.backend}: {args.batch * args.new_tokens} tokens in {time.time() - t0:.2f} s")
    for b, t in enumerate(toks):
        print(b, t)
    return 0


if __name__ == "__main__":
    sys.exit(main())
