"""FP8-aware collectives."""
from msamp.operators.dist_op.dist_op import DistOp

__all__ = ['DistOp']
