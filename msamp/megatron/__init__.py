"""Megatron-style model parallelism with FP8: tensor/sequence-parallel linears, local DDP with FP8 main grads,
the FP8 distributed optimizer and model-parallel gradient clipping.

Megatron-LM itself is optional: ``msamp.megatron.parallel_state`` provides the process-group bookkeeping
(``mpu``) when it is absent, and is used by the tests and by ``msamp.models``.
"""
from msamp.megatron import parallel_state
from msamp.megatron.layers import (
    FP8LinearWithGradAccumulationAndAsyncCommunication, ColumnParallelLinear, RowParallelLinear
)
from msamp.megatron.distributed import FP8DistributedDataParallel
from msamp.megatron.optimizer.clip_grads import clip_grad_norm_fp32
from msamp.megatron.optimizer.distrib_optimizer import FP8DistributedOptimizer

__all__ = [
    'parallel_state', 'FP8LinearWithGradAccumulationAndAsyncCommunication', 'ColumnParallelLinear', 'RowParallelLinear',
    'FP8DistributedDataParallel', 'FP8DistributedOptimizer', 'clip_grad_norm_fp32'
]
