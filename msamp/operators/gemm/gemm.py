"""Gemm.fp8_gemm with the reference's calling convention (msamp/operators/gemm/gemm.py:58-179).

``fp8_gemm(mat_a[M,K], mat_b[N,K]) -> [N,M] = mat_b · mat_aᵀ``.  The tcgen05 kernel behind it has no
multiple-of-16 constraint on M and N and zero-fills ragged K tiles in hardware, so nothing is
padded or copied (K itself must be a multiple of 16 for TMA; otherwise the operands are padded once).
``use_split_accumulator`` is accepted for compatibility: accumulation is always full fp32 in TMEM.
"""
import torch

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingTensor
from msamp.ops import gemm as _g


class Gemm:
    """Static FP8 GEMM entry point."""
    _te_base = 16

    @staticmethod
    def _round2times(value, base):
        """Smallest multiple of ``base`` that is >= ``value``."""
        return (value + base - 1) // base * base

    @classmethod
    def fp8_gemm(cls, mat_a, mat_b, out_qtype, bias=None, accumulate=False, out=None, use_split_accumulator=False):
        if not isinstance(mat_a, ScalingTensor) or not isinstance(mat_b, ScalingTensor):
            raise TypeError('fp8_gemm operands must be ScalingTensor')
        if not (Dtypes.is_fp8_qtype(mat_a.qtype) and Dtypes.is_fp8_qtype(mat_b.qtype)):
            raise TypeError('fp8_gemm operands must hold FP8 data')
        if mat_a.value.dim() != 2 or mat_b.value.dim() != 2 or mat_a.shape[1] != mat_b.shape[1]:
            raise ValueError(f'incompatible shapes {tuple(mat_a.shape)} and {tuple(mat_b.shape)}')
        out_dtype = Dtypes.get_dtype_from_qtype(out_qtype)
        if out_dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise TypeError(f'unsupported output type {out_qtype}')
        return _g.gemm_fp8(
            mat_b.value, mat_b.qtype, mat_b.meta.scale_inv, mat_a.value, mat_a.qtype, mat_a.meta.scale_inv, out_dtype, bias=bias,
            accumulate=accumulate, out=out
        )
