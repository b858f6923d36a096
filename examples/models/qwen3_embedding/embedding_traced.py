"""Qwen3-Embedding through the tracing frontend: layers and pooling are NumPy kernel functions
(`embedding_kernels/`), called directly ("numpy") or traced once per padded shape and run by the interpreter
("traced").

    python examples/models/qwen3_embedding/embedding_traced.py --layers 2 --backend traced

The serving path on the GPU is `model.py` / `example_retrieval.py` next to this file (packed sequences, paged
attention kernels).
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import Dict, List, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(_HERE, "..", "..", ".."))
sys.path.insert(0, os.path.join(_HERE, "..", "llama"))
sys.path.insert(0, _HERE)

from embedding_kernels import encoder_layer, pool_and_normalize  # noqa: E402
from llama import _np, embed  # noqa: E402

_ORDER = ["qkv_weight", "o_weight", "q_norm", "k_norm", "gate_up_weight", "down_weight", "input_norm", "post_norm"]


class TracedEmbedder:
    def __init__(self, cfg, weights: Dict, backend: str = "numpy"):
        if cfg.is_moe or not cfg.qk_norm:
            raise ValueError("this example covers dense Qwen3 layers with QK-norm")
        if backend not in ("numpy", "traced"):
            raise ValueError("backends: numpy, traced")
        self.cfg, self.backend = cfg, backend
        d = np.float32
        self.scalars = dict(n_heads=cfg.num_heads, n_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                            rope_theta=float(cfg.rope_theta), norm_eps=float(cfg.rms_eps))
        self.table, self.final_norm = _np(weights["tok_embedding"], d), _np(weights["norm_weight"], d)
        self.layers: List[Dict[str, np.ndarray]] = []
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            self.layers.append({
                "qkv_weight": _np(weights[p + "qkv_weight"], d), "o_weight": _np(weights[p + "o_weight"], d),
                "q_norm": _np(weights[p + "q_norm_weight"], d), "k_norm": _np(weights[p + "k_norm_weight"], d),
                "gate_up_weight": _np(weights[p + "gate_up_weight"], d), "down_weight": _np(weights[p + "down_weight"], d),
                "input_norm": _np(weights[p + "input_layernorm_weight"], d),
                "post_norm": _np(weights[p + "post_attention_layernorm_weight"], d)})
        self.graphs = {}

    def _run(self, name, fn, args, scalars):
        if self.backend == "numpy":
            return fn(*args, **scalars)
        from nkipy_b200.core.compile import trace
        from nkipy_b200.core.interp import evaluate

        key = (name,) + tuple(a.shape for a in args)
        if key not in self.graphs:
            self.graphs[key] = trace(fn).specialize(*[a.copy() for a in args], **scalars)
        return np.asarray(evaluate(self.graphs[key], list(args))[0])

    def encode(self, token_ids: Sequence[Sequence[int]], pad_to: int = 0) -> np.ndarray:
        """B token lists -> L2-normalised embeddings float32 [B, H]."""
        lens = [len(t) for t in token_ids]
        T = max(max(lens), pad_to)
        ids = np.zeros((len(lens), T), np.int32)
        for b, t in enumerate(token_ids):
            ids[b, :len(t)] = t
        x = embed(ids, self.table)
        for lw in self.layers:
            x = self._run("layer", encoder_layer, [x] + [lw[k] for k in _ORDER], self.scalars)
        last = np.asarray(lens, np.int32) - 1
        return self._run("pool", pool_and_normalize, [x, last, self.final_norm], dict(norm_eps=self.scalars["norm_eps"]))


def main(argv=None) -> int:
    import torch

    from nkipy_b200.models import config as C
    from nkipy_b200.models.weights import random_weights

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--backend", choices=["numpy", "traced"], default="traced")
    args = ap.parse_args(argv)
    cfg = C.tiny(hidden_size=128, head_dim=64, num_heads=2, num_kv_heads=1, vocab_size=512, num_layers=args.layers,
                 qk_norm=True, intermediate_size=256, rms_eps=1e-6)
    w = random_weights(cfg, seed=0, std=0.05, dtype=torch.float32)
    model = TracedEmbedder(cfg, w, backend=args.backend)
    rng = np.random.default_rng(0)
    docs = [rng.integers(1, cfg.vocab_size, n).tolist() for n in (5, 9, 7)]
    e = model.encode(docs)
    print("embeddings", e.shape, "norms", np.linalg.norm(e, axis=-1).round(4).tolist())
    print("similarity\n", (e @ e.T).round(3))
    return 0


if __name__ == "__main__":
    sys.exit(main())
