"""Scaling tensors: value + per-tensor scale metadata, casts, collectives and hooks."""
from msamp.common.tensor.hook import HookManager
from msamp.common.tensor.meta import ScalingMeta
from msamp.common.tensor.cast import TypeCast
from msamp.common.tensor.tensor import ScalingTensor
from msamp.common.tensor.tensor_dist import TensorDist

__all__ = ['HookManager', 'ScalingMeta', 'TypeCast', 'ScalingTensor', 'TensorDist']
