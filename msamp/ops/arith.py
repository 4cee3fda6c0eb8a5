"""FP8 accumulate and simulated-FP4 element-wise kernels (CUDA) with CPU emulations."""
import ctypes

import torch

from msamp.common.dtype import Dtypes, Floating
from msamp.ops import native
from msamp.ops import cast as _cast

_F8 = Dtypes.qtype_to_float8
_tmp = {}

E2M1_VALUES = (-6.0, -4.0, -3.0, -2.0, -1.5, -1.0, -0.5, 0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _scratch(device):
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    t = _tmp.get(key)
    if t is None:
        t = _tmp[key] = torch.zeros(1, dtype=torch.float32, device=device)
    return t


def add_to_fp8(fp8, qtype, scale, scale_inv, amax0, other):
    """In place: ``fp8 <- quantise(dequantise(fp8) + other)`` with a new scale from the amax of the sum.

    ``scale``, ``scale_inv``, ``amax0`` (0-d tensors) are updated to describe the result.
    """
    if fp8.is_cuda:
        native.check(
            native.lib().msamp_add_to_fp8(
                native.ptr(fp8), native.i64(fp8.numel()), native.fmt(qtype), native.ptr(scale), native.ptr(scale_inv), native.ptr(amax0),
                native.ptr(other), native.dt(other.dtype), native.ptr(_scratch(fp8.device)), native.stream()
            ), 'add_to_fp8'
        )
        return
    total = fp8.view(torch.uint8).view(_F8[qtype]).float() * scale_inv.float() + other.float()
    _cast.amax(total, out=amax0)
    scale.copy_(_cast.compute_scale(amax0, scale, Floating.qfp_max[qtype]))
    scale_inv.copy_(torch.reciprocal(scale))
    fp8.copy_(_cast._emulate_to_fp8(total, scale, qtype).view(fp8.dtype).view_as(fp8))


def fp4_quantize_e2m1(x):
    """Round each bf16 element to the nearest e2m1 value (ties go up)."""
    if x.is_cuda:
        x = x.contiguous()
        out = torch.empty_like(x)
        native.check(native.lib().msamp_fp4_quantize_bf16(native.ptr(x), native.ptr(out), native.i64(x.numel()), native.stream()), 'fp4_quantize')
        return out
    grid = torch.tensor(E2M1_VALUES, dtype=torch.float32)
    mids = (grid[1:] + grid[:-1]) / 2
    idx = torch.bucketize(x.float(), mids, right=True)
    return grid[idx].to(x.dtype)


def fp4_dge(x, k, clamp_max):
    """Derivative of the differentiable e2m1 quantisation surrogate, element-wise on bf16."""
    if x.is_cuda:
        x = x.contiguous()
        out = torch.empty_like(x)
        native.check(
            native.lib().msamp_fp4_dge_bf16(
                native.ptr(x), native.ptr(out), ctypes.c_float(k), ctypes.c_float(clamp_max), native.i64(x.numel()), native.stream()
            ), 'fp4_dge'
        )
        return out
    v = x.float()
    grid = torch.tensor(E2M1_VALUES, dtype=torch.float32)
    idx = (torch.bucketize(v, grid, right=True) - 1).clamp(0, 13)
    a = grid[idx]
    delta = grid[idx + 1] - a
    t = (2 * (v - a) / delta - 1).abs()
    dy = torch.clamp(t.pow(1.0 / k - 1.0) / k, max=clamp_max)
    dy = torch.where(v > 6.0, torch.zeros_like(dy), dy)
    return dy.to(x.dtype)
