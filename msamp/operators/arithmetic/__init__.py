"""Arithmetic on FP8 tensors."""
from msamp.operators.arithmetic.arithmetic import Arithmetic

__all__ = ['Arithmetic']
