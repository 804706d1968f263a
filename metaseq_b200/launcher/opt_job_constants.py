"""Published OPT model sizes and training-run constants (reference:
metaseq/launcher/opt_job_constants.py:32-45)."""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum


@dataclass
class Size:
    n_layers: int
    emb_size: int
    n_heads: int
    d_head: int
    batch_size: int  # tokens per update
    lr: float
    model_parallel: int

    @property
    def ffn_size(self):
        return 4 * self.emb_size


TOTAL_TRAIN_TOKENS = 300e9
TOTAL_WARMUP_TOKENS = 375e6
M = 1024 * 1024

# name  layers  width  heads  head-dim  batch (Mi tokens per update)  peak lr  tensor-parallel parts
_TABLE = """
8m_mp1     4    128   2   64  0.125  1.0e-3  1
8m         4    128   2   64  0.125  1.0e-3  2
125m      12    768  12   64  0.5    6.0e-4  2
350m      24   1024  16   64  0.5    3.0e-4  2
760m      24   1536  16   96  0.5    2.5e-4  2
1.3b      24   2048  32   64  1.0    2.0e-4  2
2.7b      32   2560  32   80  1.0    1.6e-4  4
6.7b      32   4096  32  128  2.0    1.2e-4  2
13b       40   5120  40  128  4.0    1.0e-4  2
30b       48   7168  56  128  4.0    1.0e-4  2
66b       64   9216  72  128  2.0    8e-5    8
175b      96  12288  96  128  2.0    3e-5    8
"""


def _parse(table: str):
    sizes = {}
    for row in table.strip().splitlines():
        name, layers, width, heads, d_head, batch_mi, lr, parts = row.split()
        size = Size(int(layers), int(width), int(heads), int(d_head), int(float(batch_mi) * M), float(lr), int(parts))
        assert size.n_heads * size.d_head == size.emb_size, name
        sizes[name] = size
    return sizes


MODEL_SIZES = _parse(_TABLE)


class ComputeEnvs(Enum):
    AWS = "aws"
    AZURE = "azure"
    FAIR = "fair"
    RSC = "rsc"
    LOCAL = "local"


DATA_LOCATIONS = {ComputeEnvs.AZURE: "/data/opt"}
DEFAULT_PARTITION = {ComputeEnvs.FAIR: "learnfair", ComputeEnvs.AZURE: None, ComputeEnvs.AWS: None,
                     ComputeEnvs.RSC: "learn", ComputeEnvs.LOCAL: None}
VALID_SUBSETS = ["BookCorpusFair", "CommonCrawl", "DM_Mathematics", "Gutenberg_PG-19", "HackerNews",
                 "OpenSubtitles", "OpenWebText2", "USPTO", "Wikipedia_en", "redditflattened", "stories"]
