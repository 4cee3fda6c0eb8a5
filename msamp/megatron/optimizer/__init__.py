"""Megatron optimizer pieces: FP8 distributed optimizer and model-parallel gradient clipping."""
from msamp.megatron.optimizer.clip_grads import clip_grad_norm_fp32
from msamp.megatron.optimizer.distrib_optimizer import FP8DistributedOptimizer

__all__ = ['clip_grad_norm_fp32', 'FP8DistributedOptimizer']
