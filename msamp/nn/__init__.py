"""Neural-network layer: FP8 linear, parameter/module types, model state, clipping, FP8 DDP."""
from msamp.nn.state import model_state
from msamp.nn.parameter import ScalingParameter
from msamp.nn.module import ScalingModule
from msamp.nn.functional import FunctionalOverider    # noqa: F401  (installs the F.linear override)
from msamp.nn.linear import FP8Linear, LinearReplacer
from msamp.nn.clip_grad import clip_grad_norm_
from msamp.nn import distributed    # noqa: F401  (installs the FP8-aware DDP class)

__all__ = ['model_state', 'ScalingParameter', 'ScalingModule', 'FP8Linear', 'LinearReplacer', 'clip_grad_norm_']
