"""Qwen3-Embedding model wrapper used by the retrieval example (reference: examples/models/qwen3_embedding/model.py)."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", ".."))

from nkipy_b200.models.embedding import EmbeddingModel  # noqa: E402
from nkipy_b200.models.weights import load_shard, random_weights  # noqa: E402


def load_model(cfg, checkpoint=None, device="cuda", max_batch=32, max_model_len=512, seed=0):
    weights = load_shard(checkpoint, 0, device=device) if checkpoint else random_weights(cfg, 0, 1, device=device,
                                                                                         seed=seed)
    return EmbeddingModel(cfg, weights, device, max_batch=max_batch, max_model_len=max_model_len)
