"""Fully sharded data parallelism (ZeRO-3 style) for FP8 models."""
from msamp.fsdp.replacer import FsdpReplacer
from msamp.fsdp.fully_sharded_data_parallel import FP8FullyShardedDataParallel, ShardedFP8Linear
from msamp.fsdp.torch_fsdp import make_fp8_comm_hook, wrap_with_torch_fsdp

__all__ = ['FsdpReplacer', 'FP8FullyShardedDataParallel', 'ShardedFP8Linear', 'wrap_with_torch_fsdp', 'make_fp8_comm_hook']
