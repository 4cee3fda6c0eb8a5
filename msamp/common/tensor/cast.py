"""Conversions between high-precision tensors and scaled low-precision payloads.

Contract (reference: msamp/common/tensor/cast.py:17-136):

* in-time scaling (window 1 or warm-up): ``amax[0] = max|x|`` → scale by the power-of-two rule → cast;
* delayed scaling: cast with the stored scale and record ``max|x|`` in ``amax[0]`` for later;
* ``sync=True``: the amax is MAX-reduced over ``meta.group`` first (NaN counted as inf) so that all
  ranks quantise with one scale;
* after every cast ``scale_inv = 1 / scale``.

The in-time path costs two kernels (amax + scale, then cast); nothing synchronises with the host.
"""
import torch
import torch.distributed as dist

from msamp.common.dtype import Dtypes
from msamp.common.utils.dist import DistUtil
from msamp import ops
from msamp.ops import cast as _k


class TypeCast:
    """Static cast helpers operating on (tensor, ScalingMeta) pairs."""
    @staticmethod
    def _prepare_scale(input, meta, sync):
        """Bring ``meta.scale``/``scale_inv``/``amax[0]`` up to date for casting ``input``.

        Returns True if the cast itself still has to record amax (delayed scaling).
        """
        in_time = meta.is_in_time_scaling()
        amax0 = meta.amax[0]
        world = DistUtil.get_world_size(meta.group) if sync else 1
        if sync and world > 1:
            if in_time:
                _k.amax(input, out=amax0)
            else:
                amax0.nan_to_num_(nan=torch.inf, posinf=torch.inf)
            dist.all_reduce(amax0, op=dist.ReduceOp.MAX, group=meta.group)
            _k.update_scales(amax0, meta.scale, meta.scale_inv, meta.qtype)
            return False
        if in_time or sync:
            if in_time:
                _k.amax_and_scale(input, amax0, meta.scale, meta.scale_inv, meta.qtype)
            else:
                _k.update_scales(amax0, meta.scale, meta.scale_inv, meta.qtype)
            return False
        return True

    @staticmethod
    def cast_to_fp8(input, meta, sync=False, fuse_transpose=False):
        """Quantise to FP8 bytes (``torch.uint8``). With ``fuse_transpose`` returns ``(out, out_t)`` of a 2-D input."""
        if input.dtype in (torch.uint8, torch.int8):
            raise TypeError('cast_to_fp8 expects a high-precision tensor')
        if meta.scale.device != input.device:
            raise ValueError(f'meta is on {meta.scale.device} but the tensor is on {input.device}')
        input = input.contiguous()
        record = TypeCast._prepare_scale(input, meta, sync)
        amax_out = meta.amax[0] if record else None
        sinv_out = meta.scale_inv if record else None
        if fuse_transpose:
            x2d = input.reshape(-1, input.shape[-1])
            out, out_t = _k.cast_transpose_fp8(x2d, meta.qtype, meta.scale, amax_out, scale_inv_out=sinv_out)
        else:
            out = _k.cast_to_fp8(input, meta.qtype, meta.scale, amax_out, scale_inv_out=sinv_out)
        return (out, out_t) if fuse_transpose else out

    @staticmethod
    def cast_to_fp16(input, meta, sync=False):
        """Scaled cast to the 16/32-bit dtype named by ``meta.qtype``: ``(x * scale).to(dtype)``."""
        in_time = meta.is_in_time_scaling()
        amax0 = meta.amax[0]
        if in_time or sync:
            _k.amax(input, out=amax0)
        if sync and DistUtil.get_world_size(meta.group) > 1:
            dist.all_reduce(amax0, op=dist.ReduceOp.MAX, group=meta.group)
        if in_time or sync:
            meta.reset_scaling_factor()
        torch.reciprocal(meta.scale, out=meta.scale_inv)
        dtype = Dtypes.get_dtype_from_qtype(meta.qtype)
        return (input.float() * meta.scale).to(dtype)    # fp32 math: a 0-d scale would not promote a half tensor

    @staticmethod
    def cast_from_fp8(input, meta, otype):
        """Dequantise FP8 bytes to the dtype of ``otype``."""
        if input.dtype != torch.uint8:
            raise ValueError('The dtype of input tensor is not torch.uint8.')
        return _k.cast_from_fp8(input.contiguous(), meta.qtype, meta.scale_inv, Dtypes.get_dtype_from_qtype(otype))

    @staticmethod
    def cast_from_fp16(input, meta, otype):
        """Undo a scaled 16/32-bit cast: ``(x * scale_inv).to(dtype)``."""
        return (input.float() * meta.scale_inv).to(Dtypes.get_dtype_from_qtype(otype))

    cast_from_fp32 = cast_from_fp16


__all__ = ['TypeCast', 'ops']
