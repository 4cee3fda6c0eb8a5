"""Simulated FP4 quantisation."""
from msamp.operators.fp4_quantize.fp4_quantize import FP4_QUANTIZER

__all__ = ['FP4_QUANTIZER']
