"""Locates the first module whose forward output or backward gradient contains NaN/Inf.

Used as a context manager around a re-run of the failing step: hooks are attached to every submodule, the
first non-finite tensor seen in each direction is reported with the module's qualified name, and on exit the
per-parameter gradient norms are logged when any of them is non-finite
(behaviour of metaseq/nan_detector.py:13-107)."""
from __future__ import annotations

import logging
from typing import Dict, Iterable, Optional

import torch

logger = logging.getLogger(__name__)


def _tensors_in(obj) -> Iterable[torch.Tensor]:
    """All tensors inside nested tuples / lists / dicts."""
    pending = [obj]
    while pending:
        x = pending.pop()
        if torch.is_tensor(x):
            yield x
        elif isinstance(x, dict):
            pending.extend(x.values())
        elif isinstance(x, (list, tuple)):
            pending.extend(x)


def _kind_of_nonfinite(t: torch.Tensor) -> Optional[str]:
    if not torch.is_floating_point(t) or t.numel() < 2:
        return None
    with torch.no_grad():
        if torch.isfinite(t).all():
            return None
        return "NaN" if torch.isnan(t).any() else "Inf"


class NanDetector:
    def __init__(self, model, forward=True, backward=True):
        self.forward, self.backward = forward, backward
        self.named_parameters = list(model.named_parameters())
        self._names: Dict[int, str] = {}
        self._handles = []
        self.reset()
        self._fhook, self._bhook = self._make_hook(False), self._make_hook(True)
        for qualified, module in model.named_modules():
            self._names[id(module)] = qualified or module.__class__.__name__
            self.add_hooks(module)

    def add_hooks(self, module):
        """Watches one more module (every submodule of the model is added at construction)."""
        self._names.setdefault(id(module), module.__class__.__name__)
        if self.forward:
            self._handles.append(module.register_forward_hook(self.fhook_fn))
        if self.backward:
            self._handles.append(module.register_full_backward_hook(self.bhook_fn))

    def fhook_fn(self, module, inp, output):
        self._fhook(module, inp, output)

    def bhook_fn(self, module, inp, output):
        self._bhook(module, inp, output)

    # has_printed_f / has_printed_b: one report per direction
    def reset(self):
        self.has_printed_f = False
        self.has_printed_b = False

    def _make_hook(self, is_backward: bool):
        flag = "has_printed_b" if is_backward else "has_printed_f"
        direction = "backward" if is_backward else "forward"

        def hook(module, inputs, outputs):
            if getattr(self, flag):
                return
            for t in _tensors_in(outputs):
                kind = _kind_of_nonfinite(t)
                if kind is None:
                    continue
                msg = (f"{kind} detected in output of {self._names.get(id(module), '?')}, "
                       f"shape: {tuple(t.shape)}, {direction}")
                first_in = next(iter(_tensors_in(inputs)), None)
                if first_in is not None and not is_backward and first_in.numel() > 0:
                    msg += f" input max: {first_in.max().item()}, input min: {first_in.min().item()}"
                logger.warning(msg)
                setattr(self, flag, True)
                return

        return hook

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc_value, exc_traceback):
        norms, bad = {}, {}
        for name, p in self.named_parameters:
            if p.grad is None:
                continue
            n = torch.linalg.vector_norm(p.grad.detach().float())
            norms[name] = n.item()
            if not torch.isfinite(n):
                bad[name] = p.grad.detach()
        if bad:
            logger.info("Detected nan/inf grad norm, dumping norms...")
            logger.info(f"norms: {norms}")
            logger.info(f"gradients: {bad}")
        self.close()

    def close(self):
        while self._handles:
            self._handles.pop().remove()
