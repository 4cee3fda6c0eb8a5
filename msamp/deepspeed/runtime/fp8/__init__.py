"""Mixed-precision optimizer wrapper with loss scaling for FP8 models (no ZeRO)."""
from msamp.deepspeed.runtime.fp8.fused_optimizer import FP8Optimizer
from msamp.deepspeed.runtime.fp8.loss_scaler import DynamicLossScaler, LossScaler

__all__ = ['FP8Optimizer', 'DynamicLossScaler', 'LossScaler']
