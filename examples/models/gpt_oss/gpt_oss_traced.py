"""gpt-oss through the tracing frontend: every layer is a NumPy kernel function (`gpt_oss_kernels/`), called
directly ("numpy") or traced once per shape and layer type and run by the IR interpreter ("traced").

    python examples/models/gpt_oss/gpt_oss_traced.py --layers 2 --experts 8 --top-k 2 -n 8

The serving path of this model on the GPU is `gpt_oss.py` next to this file.
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

from gpt_oss_kernels import decode_layer, prefill_layer  # noqa: E402
from llama import _np, embed  # noqa: E402
from llama_kernels import greedy_token  # noqa: E402

_ORDER = ["qkv_weight", "qkv_bias", "o_weight", "o_bias", "sinks", "router_weight", "router_bias", "gate_up_weight",
          "gate_up_bias", "down_weight", "down_bias", "input_norm", "post_norm", "cos", "sin", "cache_k", "cache_v"]


class TracedGptOss:
    def __init__(self, cfg, weights: Dict, batch: int, prompt_len: int, max_seq_len: int, backend: str = "numpy"):
        if not (cfg.is_moe and cfg.attn_bias and cfg.attention_sinks and cfg.router_mode == "topk_softmax"):
            raise ValueError("this example covers gpt-oss layers (biases, sinks, top-k-then-softmax routing)")
        if backend not in ("numpy", "traced"):
            raise ValueError("backends: numpy, traced")
        import torch

        from nkipy_b200.models.config import yarn_inv_freq

        self.cfg, self.batch, self.prompt_len, self.max_seq_len, self.backend = cfg, batch, prompt_len, max_seq_len, backend
        d = np.float32
        inv_freq, scale = yarn_inv_freq(cfg)
        ang = torch.arange(max_seq_len, dtype=torch.float64)[:, None] * inv_freq[None, :]
        cos, sin = (ang.cos() * scale).float().numpy(), (ang.sin() * scale).float().numpy()
        self.scalars = dict(n_heads=cfg.num_heads, n_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                            norm_eps=float(cfg.rms_eps), top_k=cfg.top_k, limit=float(cfg.swiglu_limit),
                            alpha=float(cfg.swiglu_alpha))
        self.host = {"table": _np(weights["tok_embedding"], d), "final_norm": _np(weights["norm_weight"], d),
                     "lm_head": _np(weights["lm_head_weight"], d)}
        self.layers: List[Dict[str, np.ndarray]] = []
        self.windows = [cfg.window_for_layer(i) for i in range(cfg.num_layers)]
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            lw = {k: _np(weights[p + k], d) for k in ("qkv_weight", "qkv_bias", "o_weight", "o_bias", "sinks",
                                                       "router_weight", "router_bias", "gate_up_weight", "gate_up_bias",
                                                       "down_weight", "down_bias")}
            lw.update(input_norm=_np(weights[p + "input_layernorm_weight"], d),
                      post_norm=_np(weights[p + "post_attention_layernorm_weight"], d), cos=cos, sin=sin,
                      cache_k=np.zeros((batch, max_seq_len, cfg.num_kv_heads, cfg.head_dim), d),
                      cache_v=np.zeros((batch, max_seq_len, cfg.num_kv_heads, cfg.head_dim), d))
            self.layers.append(lw)
        self.graphs = {}

    def _layer(self, which: str, x, i: int, start_pos=None):
        lw, window = self.layers[i], self.windows[i]
        args = [lw[k] for k in _ORDER]
        lead = [x] if start_pos is None else [x, start_pos]
        fn = prefill_layer if which == "prefill" else decode_layer
        if self.backend == "numpy":
            return fn(*lead, *args, window=window, **self.scalars)
        from nkipy_b200.core.compile import trace
        from nkipy_b200.core.interp import evaluate

        key = (which, window)
        if key not in self.graphs:
            self.graphs[key] = trace(fn).specialize(*[a.copy() for a in lead + args], window=window, **self.scalars)
        g = self.graphs[key]
        out = evaluate(g, lead + args)
        names = [o.name for o in g.outputs]
        lw["cache_k"], lw["cache_v"] = np.asarray(out[names.index("cache_k")]), np.asarray(out[names.index("cache_v")])
        return np.asarray(out[names.index("output0")])

    def generate(self, prompts, new_tokens: int) -> List[List[int]]:
        prompts = np.asarray(prompts, dtype=np.int32)
        B, T = prompts.shape
        if (B, T) != (self.batch, self.prompt_len) or T + new_tokens > self.max_seq_len:
            raise ValueError("prompt shape or length does not fit what the model was built for")
        eps = self.scalars["norm_eps"]
        out = [[] for _ in range(B)]
        x = embed(prompts, self.host["table"])
        for i in range(len(self.layers)):
            x = self._layer("prefill", x, i)
        tok = greedy_token(x, self.host["final_norm"], self.host["lm_head"], eps)
        for step in range(new_tokens):
            for b in range(B):
                out[b].append(int(tok[b]))
            if step + 1 == new_tokens:
                break
            x = embed(np.asarray(tok).reshape(B, 1).astype(np.int32), self.host["table"])
            pos = np.array([T + step], np.int32)
            for i in range(len(self.layers)):
                x = self._layer("decode", x, i, pos)
            tok = greedy_token(x, self.host["final_norm"], self.host["lm_head"], eps)
        return out


def tiny_config(layers: int = 2, hidden: int = 128, experts: int = 6, top_k: int = 2, window: int = 4):
    from nkipy_b200.models import config as C

    return C.tiny(hidden_size=hidden, head_dim=64, num_heads=hidden // 64, num_kv_heads=1, vocab_size=384,
                  num_layers=layers, attn_bias=True, num_experts=experts, top_k=top_k, moe_intermediate_size=hidden // 2,
                  intermediate_size=0, router_mode="topk_softmax", router_bias=True, expert_bias=True,
                  sliding_window=window,
                  layer_types=["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(layers)],
                  attention_sinks=True, swiglu_limit=7.0, swiglu_alpha=1.702, rope_scaling_factor=4.0,
                  rope_original_max_position=16, max_position=64, rope_theta=150000.0)


def main(argv=None) -> int:
    import torch

    from nkipy_b200.models.weights import random_weights

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--prompt-len", type=int, default=12)
    ap.add_argument("-n", "--new-tokens", type=int, default=8)
    ap.add_argument("--backend", choices=["numpy", "traced"], default="traced")
    args = ap.parse_args(argv)
    cfg = tiny_config(args.layers, 128, args.experts, args.top_k)
    w = random_weights(cfg, seed=0, std=0.05, dtype=torch.float32)
    model = TracedGptOss(cfg, w, args.batch, args.prompt_len, args.prompt_len + args.new_tokens, backend=args.backend)
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
