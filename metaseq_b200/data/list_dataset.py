"""Import location kept for users of the reference layout (metaseq/data/list_dataset.py)."""
from .token_transforms import ListDataset  # noqa: F401
