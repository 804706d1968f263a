"""Import location kept for users of the reference layout (metaseq/data/streaming_src_tgt_dataset.py)."""
from .streaming_blocks import (  # noqa: F401
    StreamingSrcTgtDataset,
    yield_src_tgt_blocks,
    yield_src_tgt_single_sentences_pad_8,
)
