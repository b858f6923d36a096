"""Pooling / normalisation helpers re-exported for the example scripts."""
from nkipy_b200.models.embedding import get_detailed_instruct, last_token_pool, normalize_embeddings  # noqa: F401
