"""Module base class that can own ScalingParameters."""
import torch.nn as nn

from msamp.common.tensor import ScalingTensor
from msamp.nn.parameter import ScalingParameter


class ScalingModule(nn.Module):
    """``nn.Module`` whose parameter table accepts ScalingParameter.

    ``__setattr__`` files a ScalingParameter under ``_parameters`` so that ``parameters()``,
    ``state_dict()`` and optimizers see it; ``_apply`` (behind ``.cuda()``, ``.to()``, ``.float()``…)
    hands ScalingParameters to the conversion function separately, because torch's own
    implementation only understands ``torch.Tensor``.  (reference: msamp/nn/module.py:13-93)
    """
    def __init__(self):
        super().__init__()
        self.scaling_metas = None

    def __setattr__(self, name, value):
        if isinstance(value, ScalingParameter):
            self.__dict__.pop(name, None)
            self._parameters[name] = value
        else:
            super().__setattr__(name, value)

    def _apply(self, fn, recurse=True):
        held = {k: p for k, p in self._parameters.items() if isinstance(p, ScalingParameter)}
        for k in held:
            self._parameters[k] = None
        try:
            super()._apply(fn, recurse)
        finally:
            for k, p in held.items():
                self._parameters[k] = p
        for p in held.values():
            out = fn(p)
            if out is not p and isinstance(out, ScalingTensor):
                p.data = out
            if p.grad is not None and hasattr(p.grad, 'value'):
                g = fn(p.grad)
                if g is not p.grad:
                    p.grad = g
        return self
