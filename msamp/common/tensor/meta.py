"""Per-tensor scaling state.

A ``ScalingMeta`` owns ``scale`` (multiplied in before quantising), ``scale_inv`` (multiplied in
when dequantising), a window of recent absolute maxima ``amax`` and a host-side step counter.
Attribute names follow the reference (msamp/common/tensor/meta.py:16-35) because instances are
pickled into checkpoints.  Unlike the reference the tensors live on whatever device the caller
asks for (default: the current CUDA device if there is one, else the CPU).
"""
import copy

import torch

from msamp.common.dtype import Dtypes, Floating


def _default_device():
    from msamp.common.utils.device import default_device
    return default_device()


class ScalingMeta:
    """Scale, inverse scale and amax history of one quantised tensor."""
    in_time_scaling: bool = True

    def __init__(self, qtype, scale=None, scale_inv=None, amax=None, window_size=1, group=None, device=None):
        if device is None:
            for t in (scale, scale_inv, amax):
                if t is not None:
                    device = t.device
                    break
            else:
                device = _default_device()
        self.qtype = qtype
        self.scale = scale if scale is not None else torch.ones((), device=device)
        self.scale_inv = scale_inv if scale_inv is not None else torch.ones((), device=device)
        self.amax = amax if amax is not None else torch.zeros((window_size, ), device=device)
        self.amax_counter = torch.zeros((), dtype=torch.int32)
        self.window_size = window_size
        self.group = group
        self.locked = False

    @staticmethod
    def compute_scaling_factor(amax, scale, fp_max, margin):
        """Power-of-two scale: ``2^(floor(log2(fp_max/amax)) - margin)``; ``scale`` is kept where amax is 0 or non-finite."""
        amax = amax.float()
        exp = torch.floor(torch.log2(fp_max / amax)) - margin
        sf = torch.round(torch.pow(2, torch.abs(exp)))
        sf = torch.where(amax > 0.0, sf, scale)
        sf = torch.where(torch.isfinite(amax), sf, scale)
        sf = torch.where(exp < 0, 1 / sf, sf)
        return sf

    def is_warmup(self):
        """True until ``window_size`` optimizer steps have been recorded."""
        return bool(self.amax_counter < self.window_size)

    def is_in_time_scaling(self):
        """Whether the next cast derives its scale from the tensor being cast."""
        return ScalingMeta.in_time_scaling and (self.window_size == 1 or self.is_warmup())

    @staticmethod
    def in_time_scaling_context(enabled):
        """Context manager that overrides the class-wide ``in_time_scaling`` switch."""
        class _Ctx:
            def __enter__(self):
                self.saved = ScalingMeta.in_time_scaling
                ScalingMeta.in_time_scaling = enabled

            def __exit__(self, *exc):
                ScalingMeta.in_time_scaling = self.saved

        return _Ctx()

    def reset_scaling_factor(self, qtype=None):
        """Recompute ``scale`` from ``amax[0]`` (1 for fp32/bf16, which need no scaling)."""
        qtype = self.qtype if qtype is None else qtype
        if qtype in (Dtypes.kfloat32, Dtypes.kbfloat16):
            self.scale.fill_(1)
            return
        fp_max = Floating.qfp_max[qtype]
        self.scale.copy_(ScalingMeta.compute_scaling_factor(self.amax[0], self.scale, fp_max, 0))

    def __setstate__(self, state):
        """Unpickle; a checkpoint written by the reference after a CUDA optimizer step holds ``scale`` / ``scale_inv`` as
        Python floats (msamp/optim/adamw.py:188-193): they become 0-d fp32 tensors again, next to ``amax``."""
        self.__dict__.update(state)
        amax = self.__dict__.get('amax')
        device = amax.device if torch.is_tensor(amax) else torch.device('cpu')
        for key in ('scale', 'scale_inv'):
            v = self.__dict__.get(key)
            if v is not None and not torch.is_tensor(v):
                self.__dict__[key] = torch.tensor(float(v), dtype=torch.float32, device=device)
        self.__dict__.setdefault('group', None)
        self.__dict__.setdefault('locked', False)

    def copy_(self, src):
        """Copy every field of ``src`` except group and lock."""
        self.qtype = src.qtype
        self.scale.copy_(src.scale)
        self.scale_inv.copy_(src.scale_inv)
        self.amax.copy_(src.amax)
        self.amax_counter.copy_(src.amax_counter)
        self.window_size = src.window_size
        return self

    def clone(self):
        """Deep copy sharing only the process group."""
        group, self.group = self.group, None
        try:
            obj = copy.deepcopy(self)
        finally:
            self.group = group
        obj.group = group
        obj.locked = False
        return obj

    def to(self, device):
        """Move scale, scale_inv and amax to ``device`` in place."""
        self.scale = self.scale.to(device)
        self.scale_inv = self.scale_inv.to(device)
        self.amax = self.amax.to(device)
        return self

    def cuda(self):
        return self.to(_default_device() if torch.cuda.is_available() else 'cuda')

    def cpu(self):
        return self.to('cpu')

    @property
    def is_cuda(self):
        return self.scale.is_cuda

    @property
    def device(self):
        return self.scale.device

    def __repr__(self):
        return (
            f'ScalingMeta(qtype={self.qtype}, scale={float(self.scale):g}, scale_inv={float(self.scale_inv):g}, '
            f'amax={float(self.amax.max()):g}, window_size={self.window_size})'
        )
