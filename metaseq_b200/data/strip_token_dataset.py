"""Import location kept for users of the reference layout (metaseq/data/strip_token_dataset.py)."""
from .token_transforms import StripTokenDataset  # noqa: F401
