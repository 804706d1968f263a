"""Token-embedding factory (reference layout: metaseq/modules/embedding.py); implemented in ``linear.py``."""
from .linear import Embedding  # noqa: F401
