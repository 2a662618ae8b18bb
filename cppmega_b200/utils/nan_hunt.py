"""Find where a non-finite value first appears.

``NonFiniteHunter(model)`` hangs forward (and optionally backward) hooks on every leaf-ish module and records the first
module whose output (or input gradient) contains NaN / Inf, with the step's call order, so a diverging run can be cut
down to one layer instead of bisecting launch flags by hand (the reference's NaN hunting is a set of bisect launchers:
scripts/bisect_nan_golden.sh, scripts/gb10_bisect_launcher_liger.sh).  The check is one ``isfinite().all()`` per module
output: it synchronises the device, so use it for a few diagnostic steps, not in production.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.nn as nn


def _tensors(obj):
    if torch.is_tensor(obj):
        yield obj
    elif isinstance(obj, (tuple, list)):
        for o in obj:
            yield from _tensors(o)
    elif isinstance(obj, dict):
        for o in obj.values():
            yield from _tensors(o)


class NonFiniteHunter:
    def __init__(self, model: nn.Module, backward: bool = True, only_leaves: bool = False):
        self.first: Optional[Tuple[str, str]] = None          # (phase, module name)
        self.order: List[str] = []
        self._handles = []
        for name, mod in model.named_modules():
            if not name or (only_leaves and any(True for _ in mod.children())):
                continue
            self._handles.append(mod.register_forward_hook(self._fwd(name)))
            if backward:
                self._handles.append(mod.register_full_backward_hook(self._bwd(name)))

    def _check(self, phase: str, name: str, obj) -> None:
        if self.first is not None:
            return
        for t in _tensors(obj):
            if t.is_floating_point() and t.numel() and not bool(torch.isfinite(t).all()):
                self.first = (phase, name)
                return

    def _fwd(self, name):
        def hook(_mod, _inp, out):
            self.order.append(name)
            self._check("forward", name, out)
        return hook

    def _bwd(self, name):
        def hook(_mod, grad_in, _grad_out):
            self._check("backward", name, grad_in)
        return hook

    def reset(self) -> None:
        self.first, self.order = None, []

    def close(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    def report(self) -> str:
        if self.first is None:
            return f"all {len(self.order)} module outputs finite"
        phase, name = self.first
        return f"first non-finite value: {phase} of {name!r}"
