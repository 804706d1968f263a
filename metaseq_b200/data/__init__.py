"""Data pipeline: dictionary, datasets, iterators."""
from .dictionary import Dictionary  # noqa: F401
from .base_dataset import BaseDataset, EpochListening  # noqa: F401
from . import data_utils  # noqa: F401
from .document_to_sequence import DocumentToSequenceDataset, LockingArray  # noqa: F401
from .jsonl_dataset import JsonlDataset  # noqa: F401
from .partitioned_streaming_dataset import PartitionedStreamingDataset  # noqa: F401
from .streaming_shuffle_dataset import StreamingShuffleDataset  # noqa: F401
from .concat_dataset import ConcatDataset  # noqa: F401
from .resampling_dataset import ResamplingDataset  # noqa: F401
from .synthetic import SyntheticDocumentDataset  # noqa: F401
