"""Transformer-Engine-style fused modules with FP8 ScalingParameter weights, and the replacer for TE models."""
from msamp.te.modules import MSAMPLinear, MSAMPLayerNormLinear, MSAMPLayerNormMLP, MSAMPTransformerLayer, te_available
from msamp.te.replacer import TeReplacer
from msamp.te import extension    # noqa: F401

__all__ = ['TeReplacer', 'MSAMPLinear', 'MSAMPLayerNormLinear', 'MSAMPLayerNormMLP', 'MSAMPTransformerLayer', 'te_available']
