"""Reference model families built on the FP8 layers (used by the examples, tests and benchmarks)."""
from msamp.models.gpt import GPT, GPTConfig, gpt_config
from msamp.models.gpt_parallel import ParallelGPT, vocab_parallel_cross_entropy
from msamp.models.vit import ViT, ViTConfig, vit_config

__all__ = ['GPT', 'GPTConfig', 'gpt_config', 'ParallelGPT', 'vocab_parallel_cross_entropy', 'ViT', 'ViTConfig', 'vit_config']
