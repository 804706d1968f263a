"""Deployment constants of the completions service.  Every value can be overridden by pointing
``METASEQ_SERVICE_CONSTANTS_MODULE`` at a module that defines the same names (reference:
metaseq/service/constants.py:8-64, override hook in metaseq/cli/interactive_hosted.py:38-54)."""
from __future__ import annotations

import os

MAX_SEQ_LEN = 2048
BATCH_SIZE = 2048  # silly high: the batcher below is limited by tokens, not sentences
MAX_BATCH_TOKENS = 3072
DEFAULT_PORT = 6010
MODEL_PARALLEL = 8
TOTAL_WORLD_SIZE = 8
MAX_BEAM = 16

try:
    import metaseq_internal  # noqa: F401  (site-specific paths, when present)
    from metaseq_internal.constants import CHECKPOINT_FOLDER, CHECKPOINT_LOCAL  # noqa: F401
except ImportError:
    CHECKPOINT_FOLDER = os.environ.get("METASEQ_CHECKPOINT_FOLDER", "/example/175B/reshard_no_os")
    CHECKPOINT_LOCAL = os.path.join(os.environ.get("METASEQ_CHECKPOINT_LOCAL", "/tmp/175B"), "reshard.pt")

BPE_MERGES = os.path.join(CHECKPOINT_FOLDER, "gpt2-merges.txt")
BPE_VOCAB = os.path.join(CHECKPOINT_FOLDER, "gpt2-vocab.json")
MODEL_FILE = os.path.join(CHECKPOINT_FOLDER, "reshard.pt")

LAUNCH_ARGS = [
    f"--model-parallel-size {MODEL_PARALLEL}",
    f"--distributed-world-size {TOTAL_WORLD_SIZE}",
    "--ddp-backend pytorch_ddp",
    "--task language_modeling",
    f"--bpe-merges {BPE_MERGES}",
    f"--bpe-vocab {BPE_VOCAB}",
    "--bpe hf_byte_bpe",
    f"--merges-filename {BPE_MERGES}",
    f"--vocab-filename {BPE_VOCAB}",
    f"--path {MODEL_FILE}",
    "--beam 1",
    "--distributed-port 13000",
    "--checkpoint-shard-count 1",
    f"--batch-size {BATCH_SIZE}",
    f"--buffer-size {BATCH_SIZE * MAX_SEQ_LEN}",
    f"--max-tokens {BATCH_SIZE * MAX_SEQ_LEN}",
    "/tmp",  # required "data" argument
]
INFERENCE_ARG_OVERRIDES = {}
