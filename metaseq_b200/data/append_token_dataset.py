"""Import location kept for users of the reference layout (metaseq/data/append_token_dataset.py)."""
from .token_transforms import AppendTokenDataset  # noqa: F401
