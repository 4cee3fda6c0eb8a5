"""Reductions over FP8 payloads (norms for clipping, overflow checks)."""
import ctypes

import torch

from msamp.common.dtype import Dtypes
from msamp.ops import native

_F8 = Dtypes.qtype_to_float8


def fp8_sumsq(value, qtype, out=None):
    """Sum of squares of the raw (unscaled) FP8 numbers in ``value`` as a 0-d fp32 tensor; accumulates into ``out`` if given."""
    if value.is_cuda:
        if out is None:
            out = torch.zeros((), dtype=torch.float32, device=value.device)
        v = value.contiguous()
        native.check(
            native.lib().msamp_fp8_sumsq(native.ptr(v), native.i64(v.numel()), native.fmt(qtype), native.ptr(out), native.stream()),
            'fp8_sumsq'
        )
        return out
    s = value.view(torch.uint8).view(_F8[qtype]).float().square().sum()
    if out is not None:
        out.add_(s)
        return out
    return s


def fp8_norm(value, qtype, scale_inv, norm_type=2.0):
    """p-norm of the dequantised tensor ``float(value) * scale_inv`` (2-norm uses a fused kernel on CUDA)."""
    if norm_type == 2.0:
        return fp8_sumsq(value, qtype).sqrt() * scale_inv.float().abs()
    deq = value.view(torch.uint8).view(_F8[qtype]).float()
    return torch.linalg.vector_norm(deq, norm_type) * scale_inv.float().abs()


__all__ = ['fp8_sumsq', 'fp8_norm', 'ctypes']
