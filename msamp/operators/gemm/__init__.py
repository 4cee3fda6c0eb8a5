"""FP8 GEMM operator."""
from msamp.operators.gemm.gemm import Gemm

__all__ = ['Gemm']
