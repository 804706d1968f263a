"""Positional-embedding factory (reference layout: metaseq/modules/positional_embedding.py); implemented in
``learned_positional_embedding.py``."""
from .learned_positional_embedding import PositionalEmbedding  # noqa: F401
