"""Import location kept for users of the reference layout (metaseq/data/shorten_dataset.py)."""
from .token_transforms import TruncateDataset, RandomCropDataset, maybe_shorten_dataset  # noqa: F401
