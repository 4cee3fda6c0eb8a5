"""O3 for a single process (or plain data parallelism): e4m3 model weights with scaled-fp16 master copies.

The reference reaches this layout only through its DeepSpeed integration (FP8Optimizer,
msamp/deepspeed/runtime/fp8/fused_optimizer.py:23-618).  Here ``msamp.initialize(model, opt, 'O3')``
returns this wrapper around the low-bit optimizer: the model's FP8Linear weights become e4m3 in one
flat buffer, the optimizer updates fp16 masters and re-quantises them after every step.
"""
from msamp.parallel.zero import ZeroShardedOptimizer


class FP8MasterOptimizer:
    """Optimizer facade: ``step`` / ``zero_grad`` / ``state_dict`` / ``param_groups`` over FP8 weights with fp16 masters."""
    def __init__(self, model, optimizer, group=None):
        self.model = model
        self.inner = optimizer
        self.zero = ZeroShardedOptimizer(model, optimizer, stage=1, group=group)

    @property
    def param_groups(self):
        return self.inner.param_groups

    @property
    def state(self):
        return self.inner.state

    def zero_grad(self, set_to_none=True):
        for p in self.zero.fp8_params:
            p.grad = None
        for p in self.zero.hp_params:
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()

    def step(self, closure=None):
        loss = closure() if closure is not None else None
        self.zero.reduce_and_step()
        return loss

    def all_reduce_grads(self, model):
        """Gradient exchange happens inside ``step``."""

    def state_dict(self):
        return self.zero.state_dict()

    def load_state_dict(self, sd):
        self.zero.load_state_dict(sd)
