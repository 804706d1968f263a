"""Deployment constants of the completions service.  Every value can be overridden by pointing
``METASEQ_SERVICE_CONSTANTS_MODULE`` at a module that defines the same names (reference:
metaseq/service/constants.py:8-64, override hook in metaseq/cli/interactive_hosted.py:38-54)."""
from __future__ import annotations

import os

# ---- request limits
MAX_SEQ_LEN = 2048       # prompt + generated tokens
MAX_BATCH_TOKENS = 3072  # token budget of one generation batch (the batcher is limited by tokens ...)
BATCH_SIZE = 2048        # ... so the sentence limit is set far out of reach
MAX_BEAM = 16

# ---- deployment shape
DEFAULT_PORT = 6010
MODEL_PARALLEL = 8
TOTAL_WORLD_SIZE = 8

# ---- checkpoint location: a site package may provide it, else the environment, else example paths
try:
    from metaseq_internal.constants import CHECKPOINT_FOLDER, CHECKPOINT_LOCAL  # noqa: F401
except ImportError:
    CHECKPOINT_FOLDER = os.environ.get("METASEQ_CHECKPOINT_FOLDER", "/example/175B/reshard_no_os")
    CHECKPOINT_LOCAL = os.path.join(os.environ.get("METASEQ_CHECKPOINT_LOCAL", "/tmp/175B"), "reshard.pt")


def _in_checkpoint_folder(name: str) -> str:
    return os.path.join(CHECKPOINT_FOLDER, name)


BPE_VOCAB = _in_checkpoint_folder("gpt2-vocab.json")
BPE_MERGES = _in_checkpoint_folder("gpt2-merges.txt")
MODEL_FILE = _in_checkpoint_folder("reshard.pt")


def _launch_args():
    """Command line handed to the generation parser by the service entry points; the trailing ``/tmp`` is the
    positional data argument the parser requires."""
    tokens = BATCH_SIZE * MAX_SEQ_LEN
    flags = {
        "--model-parallel-size": MODEL_PARALLEL,
        "--distributed-world-size": TOTAL_WORLD_SIZE,
        "--ddp-backend": "pytorch_ddp",
        "--task": "language_modeling",
        "--bpe-merges": BPE_MERGES,
        "--bpe-vocab": BPE_VOCAB,
        "--bpe": "hf_byte_bpe",
        "--merges-filename": BPE_MERGES,
        "--vocab-filename": BPE_VOCAB,
        "--path": MODEL_FILE,
        "--beam": 1,
        "--distributed-port": 13000,
        "--checkpoint-shard-count": 1,
        "--batch-size": BATCH_SIZE,
        "--buffer-size": tokens,
        "--max-tokens": tokens,
    }
    return [f"{k} {v}" for k, v in flags.items()] + ["/tmp"]


LAUNCH_ARGS = _launch_args()
INFERENCE_ARG_OVERRIDES = {}
