"""Kernel entry points under the names the reference's Transformer Engine adaptor exposes.

The reference forwards these calls to ``transformer_engine_extensions``
(msamp/common/utils/transformer_engine_wrapper.py:63-176); here they land on msamp's own sm_100a kernels
(or their CPU emulation), so code written against ``TransformerEngineWrapper`` keeps working without
Transformer Engine.  No padding to multiples of 16 is needed by these kernels.
"""
import torch

from msamp.common.dtype import Dtypes
from msamp.ops import cast as _k
from msamp.ops import gemm as _g


class TransformerEngineWrapper:
    """Static FP8 GEMM / cast / transpose helpers."""
    @staticmethod
    def _to_te_dtype(qtype):
        """Name of the equivalent Transformer Engine ``DType`` member (``kFloat8E4M3`` …)."""
        return qtype.name

    @staticmethod
    def _to_compatible_args(args):
        """Replace every QType in ``args`` by its Transformer Engine dtype name."""
        return [TransformerEngineWrapper._to_te_dtype(a) if isinstance(a, Dtypes.kbyte.__class__) else a for a in args]

    @staticmethod
    def te_gemm(A, A_scale_inv, A_type, transa, B, B_scale_inv, B_type, transb, D, D_scale, D_type, D_amax, bias, bias_type, pre_gelu_out,
                grad, workspace, workspace_size, accumulate, use_split_accumulator, math_sm_count=0):
        """cuBLASLt-style call in column-major terms: with ``transa=True, transb=False`` computes ``D = B · Aᵀ`` (row-major)."""
        if not transa or transb:
            raise NotImplementedError('only the TN layout (transa=True, transb=False) is provided')
        out_dtype = D.dtype
        has_bias = bias is not None and bias.numel() > 0
        return _g.gemm_fp8(B, B_type, B_scale_inv, A, A_type, A_scale_inv, out_dtype, bias=bias if has_bias else None,
                           accumulate=accumulate, out=D)

    @staticmethod
    def cast_to_fp8(input, scale, amax, scale_inv, otype):
        """``out = saturate(input * scale)`` in format ``otype``; ``amax`` receives ``max|input|``, ``scale_inv`` ``1/scale``."""
        return _k.cast_to_fp8(input.contiguous(), otype, scale, amax_out=amax, scale_inv_out=scale_inv)

    @staticmethod
    def cast_from_fp8(input, scale_inv, itype, otype):
        return _k.cast_from_fp8(input.contiguous(), itype, scale_inv, Dtypes.get_dtype_from_qtype(otype))

    @staticmethod
    def fp8_fused_cast_transpose(input, qtype, meta):
        """Returns ``(cast, cast transposed)`` of a 2-D tensor using ``meta.scale``; records amax and scale_inv in ``meta``."""
        x = input.reshape(-1, input.shape[-1])
        return _k.cast_transpose_fp8(x, qtype, meta.scale, amax_out=meta.amax[0], scale_inv_out=meta.scale_inv)

    @staticmethod
    def fp8_transpose(input):
        """Transpose of a 2-D FP8 ScalingTensor (shares its meta)."""
        return input.fp8_transpose()


__all__ = ['TransformerEngineWrapper', 'torch']
