"""Import location kept for users of the reference layout (metaseq/data/prepend_token_dataset.py)."""
from .token_transforms import PrependTokenDataset  # noqa: F401
