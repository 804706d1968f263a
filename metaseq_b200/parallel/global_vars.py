"""Named, reusable device buffers for collectives whose output is consumed immediately (the all-gathered
activations of sequence parallelism): one allocation per ``(name, dtype)`` that grows to the largest request
(reference: metaseq/modules/megatron/global_vars.py:53-74)."""
from __future__ import annotations

import math
from typing import Dict, Tuple

import torch

_GLOBAL_MEMORY_BUFFER = None


class GlobalMemoryBuffer:
    def __init__(self):
        self.buffer: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}

    def get_tensor(self, tensor_shape, dtype, name, device=None):
        need = math.prod(tensor_shape)
        key = (name, dtype)
        buf = self.buffer.get(key)
        if buf is None or buf.numel() < need:
            if device is None:
                device = torch.cuda.current_device() if torch.cuda.is_available() else "cpu"
            buf = torch.empty(need, dtype=dtype, device=device, requires_grad=False)
            self.buffer[key] = buf
        return buf[:need].view(*tensor_shape)


def get_global_memory_buffer() -> GlobalMemoryBuffer:
    global _GLOBAL_MEMORY_BUFFER
    if _GLOBAL_MEMORY_BUFFER is None:
        _GLOBAL_MEMORY_BUFFER = GlobalMemoryBuffer()
    return _GLOBAL_MEMORY_BUFFER
