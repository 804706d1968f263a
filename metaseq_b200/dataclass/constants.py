"""Choice lists used by the config dataclasses (flag values are the reference's:
metaseq/dataclass/constants.py:32-64)."""
from __future__ import annotations

LOG_FORMAT_CHOICES = ("json", "none")
DDP_BACKEND_CHOICES = ("c10d", "fully_sharded", "pytorch_ddp")
TASK_DDP_BACKEND_CHOICES = ("none", "c10d", "fully_sharded", "pytorch_ddp")
DATASET_IMPL_CHOICES = ("raw", "lazy", "cached", "mmap", "fasta")
CLIP_GRAD_NORM_TYPE_CHOICES = ("l2", "inf")
ATTN_CHOICES = ("math", "flash", "xformers_default")

# value of --self-attn-doc-sep meaning "no document-separator attention masking"
UNSPECIFIED_DOC_SEP = -1
