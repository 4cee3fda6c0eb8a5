"""Reference model families built on the FP8 layers (used by the examples, tests and benchmarks)."""
from msamp.models.gpt import GPT, GPTConfig, gpt_config

__all__ = ['GPT', 'GPTConfig', 'gpt_config']
