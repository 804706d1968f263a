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
MODEL_SIZES = {
    "8m_mp1": Size(4, 128, 2, 64, int(0.125 * M), 1.0e-3, 1),
    "8m": Size(4, 128, 2, 64, int(0.125 * M), 1.0e-3, 2),
    "125m": Size(12, 768, 12, 64, int(0.5 * M), 6.0e-4, 2),
    "350m": Size(24, 1024, 16, 64, int(0.5 * M), 3.0e-4, 2),
    "760m": Size(24, 1536, 16, 96, int(0.5 * M), 2.5e-4, 2),
    "1.3b": Size(24, 2048, 32, 64, int(1.0 * M), 2.0e-4, 2),
    "2.7b": Size(32, 2560, 32, 80, int(1.0 * M), 1.6e-4, 4),
    "6.7b": Size(32, 4096, 32, 128, int(2.0 * M), 1.2e-4, 2),
    "13b": Size(40, 5120, 40, 128, int(4.0 * M), 1.0e-4, 2),
    "30b": Size(48, 7168, 56, 128, int(4.0 * M), 1.0e-4, 2),
    "66b": Size(64, 9216, 72, 128, int(2.0 * M), 8e-5, 8),
    "175b": Size(96, 12288, 96, 128, int(2.0 * M), 3e-5, 8),
}
for _name, _size in MODEL_SIZES.items():
    assert _size.n_heads * _size.d_head == _size.emb_size, _name


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
