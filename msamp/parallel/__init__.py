"""Multi-GPU building blocks: data-parallel trainer, ZeRO sharding, symmetric memory and fused collectives."""
from msamp.parallel.trainer import DataParallelTrainer

__all__ = ['DataParallelTrainer']
