"""Retrieval demo: embed queries and documents, rank documents by cosine similarity
(reference: examples/models/qwen3_embedding/example_retrieval.py:60-397).

With `--model` (a Hugging Face directory with a tokenizer) and `--checkpoint` the texts below are
embedded with the real model.  Offline the script uses random weights and a deterministic word-hash
tokenizer: the scores are then meaningless, but the run exercises the same device path and checks it
against the plain PyTorch implementation (cosine between the two implementations' embeddings).
"""
import argparse
import os
import sys
import time
import zlib

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", ".."))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from model import load_model  # noqa: E402

from nkipy_b200.models.config import qwen3_embedding  # noqa: E402
from nkipy_b200.models.embedding import get_detailed_instruct, normalize_embeddings  # noqa: E402
from nkipy_b200.models.reference import EagerTransformer  # noqa: E402

TASK = "Given a web search query, retrieve relevant passages that answer the query"
QUERIES = ["What is the capital of China?", "Explain gravity"]
DOCUMENTS = [
    "The capital of China is Beijing.",
    "Gravity is a force that attracts two bodies towards each other. It gives weight to physical objects.",
    "Paged key-value caches let a serving engine share prompt prefixes between requests.",
]


def hash_tokenize(text, vocab):
    return [zlib.crc32(w.encode()) % vocab for w in text.lower().split()] or [0]


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--size", choices=["0.6b", "8b"], default="0.6b")
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--model", default=None, help="Hugging Face directory (tokenizer)")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--max-model-len", type=int, default=128)
    args = ap.parse_args()
    cfg = qwen3_embedding(args.size)
    if args.layers:
        cfg.num_layers = args.layers
    model = load_model(cfg, args.checkpoint, args.device, max_model_len=args.max_model_len)
    if args.model:
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(args.model)
        enc = lambda t: tok(t)["input_ids"]
    else:
        enc = lambda t: hash_tokenize(t, cfg.vocab_size)
    texts = [get_detailed_instruct(TASK, q) for q in QUERIES] + DOCUMENTS
    ids = [enc(t) for t in texts]
    model.encode(ids[:1])                                            # warm-up
    t0 = time.perf_counter()
    emb = model.encode(ids)
    if torch.cuda.is_available() and args.device.startswith("cuda"):
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    scores = emb[:len(QUERIES)] @ emb[len(QUERIES):].T
    print(f"embedded {len(texts)} texts ({sum(map(len, ids))} tokens) in {dt * 1e3:.1f} ms")
    for q, row in zip(QUERIES, scores.tolist()):
        print(f"{q!r}: " + ", ".join(f"{s:.3f}" for s in row))
    # cross-check against the plain PyTorch implementation
    ref = EagerTransformer(cfg, model.lm_weights if hasattr(model, "lm_weights") else _weights_of(model),
                           device=args.device, dtype=torch.bfloat16)
    ref_emb = []
    for t in ids:
        ref.reset()
        h = ref.forward(torch.tensor([t[: args.max_model_len]], device=args.device))[:, -1]
        ref_emb.append(h.float()[0])
    ref_emb = normalize_embeddings(torch.stack(ref_emb))
    cos = (emb.to(ref_emb.device) * ref_emb).sum(-1)
    print(f"cosine(ours, eager) per text: min {cos.min().item():.4f}")


def _weights_of(model):
    """Rebuild the ``x @ W`` weight dict the eager implementation expects from the loaded model."""
    lm = model.lm
    w = {"tok_embedding": lm.tok_embedding, "norm_weight": lm.final_norm, "lm_head_weight": lm.lm_head.t()}
    for i, lw in enumerate(lm.layers):
        p = f"layers.{i}."
        w[p + "qkv_weight"], w[p + "o_weight"] = lw.qkv.t(), lw.o.t()
        w[p + "gate_up_weight"], w[p + "down_weight"] = lw.gate_up.t(), lw.down.t()
        w[p + "input_layernorm_weight"], w[p + "post_attention_layernorm_weight"] = lw.input_norm, lw.post_norm
        if lw.q_norm is not None:
            w[p + "q_norm_weight"], w[p + "k_norm_weight"] = lw.q_norm, lw.k_norm
    return w


if __name__ == "__main__":
    main()
