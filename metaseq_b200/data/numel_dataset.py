"""Import location kept for users of the reference layout (metaseq/data/numel_dataset.py)."""
from .token_transforms import NumelDataset  # noqa: F401
