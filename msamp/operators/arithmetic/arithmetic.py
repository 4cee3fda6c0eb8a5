"""Arithmetic.add_to_fp8 (reference: msamp/operators/arithmetic/arithmetic.py:12-35)."""
import torch

from msamp.common.dtype import Dtypes
from msamp.ops import arith as _a


class Arithmetic:
    """Arithmetic operators for FP8 payloads."""
    @staticmethod
    def add_to_fp8(fp8_tensor, meta, other):
        """Accumulate a high-precision tensor into an FP8 tensor in place, refreshing ``meta`` (scale, scale_inv, amax[0])."""
        if fp8_tensor.dtype not in (torch.uint8, torch.int8):
            raise ValueError('The fp8 tensor is not in uint8 or int8.')
        if not Dtypes.is_fp8_qtype(meta.qtype):
            raise ValueError('The fp8 tensor is not in e4m3 or e5m2 format.')
        if not (fp8_tensor.is_contiguous() and other.is_contiguous()):
            raise ValueError('add_to_fp8 needs contiguous tensors.')
        if fp8_tensor.numel() != other.numel() or fp8_tensor.device != other.device:
            raise ValueError('add_to_fp8 needs tensors of the same size on the same device.')
        _a.add_to_fp8(fp8_tensor, meta.qtype, meta.scale, meta.scale_inv, meta.amax[0], other)
