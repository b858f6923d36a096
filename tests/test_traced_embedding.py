"""Qwen3-Embedding as NumPy kernel functions (examples/models/qwen3_embedding/embedding_kernels): padded batch,
no cache, last-token pooling and L2 normalisation -- direct and traced + interpreted, against the eager fp32 model
run on each sequence alone (so that padding cannot help or hurt)."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "examples", "models", "llama"))
sys.path.insert(0, os.path.join(ROOT, "examples", "models", "qwen3_embedding"))

from embedding_traced import TracedEmbedder  # noqa: E402

from nkipy_b200.models import config as C  # noqa: E402
from nkipy_b200.models.embedding import normalize_embeddings  # noqa: E402
from nkipy_b200.models.reference import EagerTransformer  # noqa: E402
from nkipy_b200.models.weights import random_weights  # noqa: E402


def _setup():
    cfg = C.tiny(hidden_size=128, head_dim=64, num_heads=2, num_kv_heads=1, vocab_size=512, num_layers=2, qk_norm=True,
                 intermediate_size=256, rms_eps=1e-6)
    w = random_weights(cfg, seed=5, std=0.08, dtype=torch.float32)
    for i in range(cfg.num_layers):
        g = torch.Generator().manual_seed(50 + i)
        w[f"layers.{i}.q_norm_weight"] = 1.0 + 0.2 * torch.randn(64, generator=g)
        w[f"layers.{i}.k_norm_weight"] = 1.0 + 0.2 * torch.randn(64, generator=g)
    rng = np.random.default_rng(3)
    docs = [rng.integers(1, cfg.vocab_size, n).tolist() for n in (4, 11, 7, 1)]
    ref = EagerTransformer(cfg, w, dtype=torch.float32)
    want = []
    for d in docs:
        ref.reset()
        want.append(ref.forward(torch.tensor([d]))[0, -1])
    return cfg, w, docs, normalize_embeddings(torch.stack(want)).numpy()


def test_direct_and_traced_embeddings_match_the_eager_model():
    cfg, w, docs, want = _setup()
    for backend in ("numpy", "traced"):
        model = TracedEmbedder(cfg, w, backend=backend)
        got = model.encode(docs)
        assert got.shape == want.shape and got.dtype == np.float32
        np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-5)
        np.testing.assert_allclose(np.linalg.norm(got, axis=-1), 1.0, rtol=1e-5)


def test_padding_does_not_change_an_embedding():
    cfg, w, docs, want = _setup()
    model = TracedEmbedder(cfg, w, backend="traced")
    a = model.encode(docs)
    b = model.encode(docs, pad_to=16)
    np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-6)
    assert len(model.graphs) == 4                       # layer and pooling graphs for the two padded lengths
