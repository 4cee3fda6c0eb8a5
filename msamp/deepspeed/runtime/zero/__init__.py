"""ZeRO stage 1/2 optimizer for FP8 models."""
from msamp.deepspeed.runtime.zero.fp8_stage_1_and_2 import FP8DeepSpeedZeroOptimizer
from msamp.deepspeed.runtime.zero.utils import is_zero_supported_optimizer

__all__ = ['FP8DeepSpeedZeroOptimizer', 'is_zero_supported_optimizer']
