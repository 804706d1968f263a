"""Import location kept for users of the reference layout (metaseq/data/pad_dataset.py)."""
from .token_transforms import PadDataset, LeftPadDataset, RightPadDataset, MultiplePadDataset  # noqa: F401
