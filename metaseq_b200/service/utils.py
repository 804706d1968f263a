"""Small helpers of the service layer (reference: metaseq/service/utils.py:12-17)."""
from __future__ import annotations

import logging
import re
import sys


def normalize_newlines(s: str) -> str:
    """Windows (CRLF) and old Mac (CR) line ends become LF, as the tokenizer was trained on."""
    return re.sub(r"\r\n|\r", "\n", s)


def build_logger():
    logging.basicConfig(format="%(asctime)s | %(levelname)s | %(name)s | %(message)s", datefmt="%Y-%m-%d %H:%M:%S",
                        level=logging.INFO, stream=sys.stdout)
    return logging.getLogger("metaseq_b200.cli.interactive")


def encode_fn(generator, x):
    return generator.encode_fn(x)
