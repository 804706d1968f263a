"""Import location kept for users of the reference layout (metaseq/data/sort_dataset.py)."""
from .token_transforms import SortDataset  # noqa: F401
