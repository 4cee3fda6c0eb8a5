"""Overflow detection that understands ScalingTensor (reference: msamp/deepspeed/runtime/utils.py:11-26)."""
import torch
import torch.distributed as dist

from msamp.common.tensor import ScalingTensor


class MSAMPCheckOverflow:
    """``check(params)`` → True if any gradient holds inf/nan on any rank of ``group``."""
    def __init__(self, group=None, mpu=None):
        self.group, self.mpu = group, mpu

    @staticmethod
    def _has_inf_or_nan(x):
        if isinstance(x, ScalingTensor):
            return ~torch.isfinite(x.meta.amax[0])
        s = x.float().sum()
        return ~torch.isfinite(s)

    def has_overflow(self, grads):
        flags = [self._has_inf_or_nan(g).reshape(1).float() for g in grads if g is not None]
        if not flags:
            return False
        flag = torch.cat([f.to(flags[0].device) for f in flags]).max().reshape(1)
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        if self.mpu is not None and hasattr(self.mpu, 'get_model_parallel_group'):
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.mpu.get_model_parallel_group())
        return bool(flag.item() > 0)

    def check(self, params):
        return self.has_overflow([getattr(p, 'grad', None) for p in params])
