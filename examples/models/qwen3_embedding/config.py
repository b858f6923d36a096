"""Model shapes of the Qwen3-Embedding example (reference: examples/models/qwen3_embedding/config.py:15-112)."""
from nkipy_b200.models.config import qwen3_embedding


def get_config(size: str = "0.6b"):
    return qwen3_embedding(size)
