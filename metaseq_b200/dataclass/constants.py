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


# --- enum forms, for code that builds its own choice types the way the reference does (:10-35, :59-61)
from enum import Enum, EnumMeta  # noqa: E402
from typing import Iterable  # noqa: E402


class StrEnumMeta(EnumMeta):
    """``isinstance`` check by name, so that an enum rebuilt after pickling still counts as a choice enum."""

    @classmethod
    def __instancecheck__(cls, other):
        return "enum" in str(type(other))


class StrEnum(Enum, metaclass=StrEnumMeta):
    """An enum whose members print, hash and compare as their string values."""

    def __str__(self):
        return self.value

    def __eq__(self, other):
        return self.value == (other.value if isinstance(other, Enum) else other)

    def __repr__(self):
        return self.value

    def __hash__(self):
        return hash(str(self))


def ChoiceEnum(choices: Iterable[str]):
    """An enum type with one member per allowed string."""
    return StrEnum("Choices", {k: k for k in choices})


class AttentionVariants(str, Enum):
    DEFAULT = "default"
    XFORMERS = "xformers_default"
