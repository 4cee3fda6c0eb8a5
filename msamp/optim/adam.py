"""Adam flavours (L2 regularisation instead of decoupled decay) and the DeepSpeed-style signature.

(reference: msamp/optim/adam.py:9-94)
"""
from msamp.optim.adamw import LBAdamW, FSDPAdamW


class LBAdam(LBAdamW):
    """Adam with L2 weight decay folded into the gradient."""
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, amsgrad=False, maximize=False, *args, **kwargs):
        super().__init__(params, *args, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad, maximize=maximize, **kwargs)
        self.use_adam = True


class DSAdam(LBAdamW):
    """Same constructor surface as DeepSpeed's FusedAdam (``adam_w_mode``, ``set_grad_none``)."""
    def __init__(
        self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, adam_w_mode=True, weight_decay=0., amsgrad=False,
        set_grad_none=True, **kwargs
    ):
        super().__init__(
            params, lr=lr, bias_correction=bias_correction, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad, **kwargs
        )
        self.use_adam = not adam_w_mode
        self.set_grad_none = set_grad_none


class FSDPAdam(FSDPAdamW):
    """FSDPAdamW with L2 weight decay."""
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, amsgrad=False, maximize=False, *args, **kwargs):
        super().__init__(params, *args, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad, maximize=maximize, **kwargs)
        self.use_adam = True
