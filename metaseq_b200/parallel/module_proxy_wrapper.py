"""Makes a wrapper module (for instance DistributedDataParallel) look like the module it wraps: unknown
attributes are looked up on the wrapper and then on the wrapped module, and ``state_dict`` /
``load_state_dict`` address the wrapped module directly so checkpoints carry no ``module.`` prefix
(reference: metaseq/distributed/module_proxy_wrapper.py:9-56)."""
from __future__ import annotations

from torch import nn


class ModuleProxyWrapper(nn.Module):
    def __init__(self, module: nn.Module):
        super().__init__()
        if not hasattr(module, "module"):
            raise AssertionError("ModuleProxyWrapper expects input to wrap another module")
        self.module = module

    @property
    def _innermost(self) -> nn.Module:
        return self.module.module

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def __getattr__(self, name):
        # nn.Module.__getattr__ covers parameters, buffers and submodules registered on the proxy itself
        for lookup in (lambda: nn.Module.__getattr__(self, name), lambda: getattr(self.module, name)):
            try:
                return lookup()
            except AttributeError:
                continue
        return getattr(self._innermost, name)

    def load_state_dict(self, *args, **kwargs):
        return self._innermost.load_state_dict(*args, **kwargs)

    def state_dict(self, *args, **kwargs):
        return self._innermost.state_dict(*args, **kwargs)
