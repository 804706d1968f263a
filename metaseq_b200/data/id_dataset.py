"""Import location kept for users of the reference layout (metaseq/data/id_dataset.py)."""
from .token_transforms import IdDataset  # noqa: F401
