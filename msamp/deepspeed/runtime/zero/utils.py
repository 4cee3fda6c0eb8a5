"""Which optimizers may be sharded (reference: msamp/deepspeed/runtime/zero/utils.py:6-12)."""
from msamp.optim import DSAdam, LBAdam, LBAdamW

ZERO_SUPPORTED_OPTIMIZERS = [LBAdam, LBAdamW, DSAdam]


def is_zero_supported_optimizer(optimizer):
    """True for the low-bit Adam family."""
    return type(optimizer) in ZERO_SUPPORTED_OPTIMIZERS
