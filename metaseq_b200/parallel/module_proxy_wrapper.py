"""Forwards attribute access, ``state_dict`` and ``load_state_dict`` through a wrapper module
(e.g. DDP) to the module it wraps, so callers can treat both alike (reference:
metaseq/distributed/module_proxy_wrapper.py:9-56)."""
from __future__ import annotations

from torch import nn


class ModuleProxyWrapper(nn.Module):
    def __init__(self, module: nn.Module):
        super().__init__()
        assert hasattr(module, "module"), "ModuleProxyWrapper expects input to wrap another module"
        self.module = module

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            try:
                return getattr(self.module, name)
            except AttributeError:
                return getattr(self.module.module, name)

    def state_dict(self, *args, **kwargs):
        return self.module.module.state_dict(*args, **kwargs)

    def load_state_dict(self, *args, **kwargs):
        return self.module.module.load_state_dict(*args, **kwargs)

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)
