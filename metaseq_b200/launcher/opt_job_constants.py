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

# One row per published size.  Columns: name | tensor-parallel parts | peak learning rate in units of 1e-5 |
# tokens per update in Ki | attention heads | model width | layers.  The head size is width / heads.
_TABLE = """
8m_mp1  1  100   128   2    128   4
8m      2  100   128   2    128   4
125m    2   60   512  12    768  12
350m    2   30   512  16   1024  24
760m    2   25   512  16   1536  24
1.3b    2   20  1024  32   2048  24
2.7b    4   16  1024  32   2560  32
6.7b    2   12  2048  32   4096  32
13b     2   10  4096  40   5120  40
30b     2   10  4096  56   7168  48
66b     8    8  2048  72   9216  64
175b    8    3  2048  96  12288  96
"""


def _parse(table: str):
    sizes = {}
    for row in table.strip().splitlines():
        name, parts, lr_e5, batch_ki, heads, width, layers = row.split()
        heads, width = int(heads), int(width)
        assert width % heads == 0, name
        sizes[name] = Size(n_layers=int(layers), emb_size=width, n_heads=heads, d_head=width // heads,
                           batch_size=int(batch_ki) * 1024, lr=float(lr_e5 + "e-5"), model_parallel=int(parts))
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
