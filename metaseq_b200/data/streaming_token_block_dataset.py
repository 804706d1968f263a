"""Import location kept for users of the reference layout (metaseq/data/streaming_token_block_dataset.py)."""
from .streaming_blocks import (  # noqa: F401
    StreamingTokenBlockDataset,
    yield_doc_blocks,
    yield_single_sentences_pad_8,
    yield_token_blocks,
)
