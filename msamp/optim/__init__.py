"""Low-bit optimizers."""
from msamp.optim.optimizer import LBOptimizer
from msamp.optim.adamw_base import LBAdamWBase
from msamp.optim.adamw import LBAdamW, FSDPAdamW
from msamp.optim.adam import LBAdam, DSAdam, FSDPAdam

__all__ = ['LBOptimizer', 'LBAdam', 'LBAdamW', 'DSAdam', 'LBAdamWBase', 'FSDPAdamW', 'FSDPAdam']
