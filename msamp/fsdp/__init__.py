"""Fully sharded data parallelism (ZeRO-3 style) for FP8 models."""
from msamp.fsdp.replacer import FsdpReplacer
from msamp.fsdp.fully_sharded_data_parallel import FP8FullyShardedDataParallel, ShardedFP8Linear

__all__ = ['FsdpReplacer', 'FP8FullyShardedDataParallel', 'ShardedFP8Linear']
