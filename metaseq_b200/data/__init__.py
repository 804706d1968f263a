"""Data pipeline: dictionary, datasets, iterators."""
from .dictionary import Dictionary, TruncatedDictionary  # noqa: F401
from .base_dataset import BaseDataset, EpochListening  # noqa: F401
from . import data_utils  # noqa: F401
from .document_to_sequence import DocumentToSequenceDataset, LockingArray  # noqa: F401
from .jsonl_dataset import JsonlDataset  # noqa: F401
from .partitioned_streaming_dataset import PartitionedStreamingDataset  # noqa: F401
from .streaming_shuffle_dataset import StreamingShuffleDataset  # noqa: F401
from .concat_dataset import ConcatDataset  # noqa: F401
from .resampling_dataset import ResamplingDataset  # noqa: F401
from .synthetic import SyntheticDocumentDataset  # noqa: F401
from .base_wrapper_dataset import BaseWrapperDataset  # noqa: F401,E402
from .token_transforms import (  # noqa: F401,E402
    AppendTokenDataset, IdDataset, LeftPadDataset, ListDataset, NumelDataset, PadDataset, PrependTokenDataset,
    RandomCropDataset, RightPadDataset, SortDataset, StripTokenDataset, TruncateDataset,
)
from .nested_dictionary_dataset import NestedDictionaryDataset  # noqa: F401,E402
from .token_block_dataset import TokenBlockDataset  # noqa: F401,E402
from .monolingual_dataset import MonolingualDataset  # noqa: F401,E402
from .lm_context_window_dataset import LMContextWindowDataset  # noqa: F401,E402
from .indexed_dataset import (  # noqa: F401,E402
    IndexedCachedDataset, IndexedDataset, IndexedRawTextDataset, MMapIndexedDataset,
)
from .streaming_blocks import StreamingSrcTgtDataset, StreamingTokenBlockDataset  # noqa: F401,E402
from .cm3_dataset import CausalMaskedDocumentToSequenceDataset  # noqa: F401,E402


# Names that the reference exports at package level, resolved on first use (importing them eagerly here would pull
# the kernel loader and the parallel layers into every ``import metaseq_b200.data``).
_LAZY = {
    "CountingIterator": (".iterators", "CountingIterator"),
    "EpochBatchIterator": (".iterators", "EpochBatchIterator"),
    "GroupedIterator": (".iterators", "GroupedIterator"),
    "ShardedIterator": (".iterators", "ShardedIterator"),
    "StreamingEpochBatchIterator": (".iterators", "StreamingEpochBatchIterator"),
    "MultiplePadDataset": (".token_transforms", "MultiplePadDataset"),
}


def __getattr__(name):
    try:
        module, attr = _LAZY[name]
    except KeyError:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
    import importlib

    value = getattr(importlib.import_module(module, __name__), attr)
    globals()[name] = value
    return value


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
