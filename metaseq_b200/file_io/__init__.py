"""Path abstraction: local paths natively, ``s3://`` and Azure blob URLs through optional
handlers when their SDKs are installed (reference: metaseq/file_io/__init__.py:11-64 and the
iopath-style manager in metaseq/file_io/common/)."""
from __future__ import annotations

import logging
import os
import shutil
from typing import IO, Any, Callable, Dict, List, Optional

import torch

from .path_manager import NativePathHandler, PathHandler, PathManagerBase
from .non_blocking_io import NonBlockingIOManager  # noqa: F401

logger = logging.getLogger(__name__)

PathManager = PathManagerBase()

try:
    from .s3 import S3PathHandler

    PathManager.register_handler(S3PathHandler())
except Exception:  # boto3 missing
    pass
try:
    from .azure_blob import AzureBlobPathHandler

    PathManager.register_handler(AzureBlobPathHandler())
except Exception:  # azure sdk missing
    pass


def recursively_cast_dictconfigs(cfg):
    """Config nodes saved by other tools (mapping-like objects) become plain dicts."""
    if isinstance(cfg, dict):
        return {k: recursively_cast_dictconfigs(v) for k, v in cfg.items()}
    if hasattr(cfg, "items") and not isinstance(cfg, dict) and cfg.__class__.__name__ == "DictConfig":
        return {k: recursively_cast_dictconfigs(v) for k, v in cfg.items()}
    return cfg


def torch_load_cpu(path):
    with PathManager.open(path, "rb") as f:
        state = torch.load(f, map_location=torch.device("cpu"), weights_only=False)
    if isinstance(state, dict) and "cfg" in state:
        state["cfg"] = recursively_cast_dictconfigs(state["cfg"])
        if isinstance(state["cfg"], dict) and state["cfg"].get("model") is not None \
                and isinstance(state["cfg"]["model"], dict) and "arch" in state["cfg"]["model"] and False:
            pass
    return state


def load_and_pop_last_optimizer_state(pth):
    st = torch_load_cpu(pth)
    st.pop("last_optimizer_state", None)
    return st
