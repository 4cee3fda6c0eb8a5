"""AdamW with low-bit states written with plain torch operations.

This is the numerical definition that the fused CUDA kernel follows and the oracle it is tested
against: moments are dequantised, updated in fp32, the parameter is updated with the *unquantised*
new moments, then everything is stored back in its low-precision format with a fresh per-tensor
scale.  (reference: msamp/optim/adamw_base.py:17-309)
"""
import math

import torch

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingTensor
from msamp.optim.optimizer import LBOptimizer


class LBAdamWBase(LBOptimizer):
    """Reference implementation; ``exp_avg_dtype`` / ``exp_avg_sq_dtype`` choose the state formats.

    ``torch.uint8`` → e4m3, ``torch.int8`` → e5m2, ``torch.float16`` → scaled fp16, ``torch.float32`` → plain.
    """
    def __init__(
        self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, amsgrad=False, *,
        maximize=False, exp_avg_dtype=torch.uint8, exp_avg_sq_dtype=torch.float16
    ):
        if not 0.0 <= lr:
            raise ValueError(f'Invalid learning rate: {lr}')
        if not 0.0 <= eps:
            raise ValueError(f'Invalid epsilon value: {eps}')
        if not 0.0 <= betas[0] < 1.0:
            raise ValueError(f'Invalid beta parameter at index 0: {betas[0]}')
        if not 0.0 <= betas[1] < 1.0:
            raise ValueError(f'Invalid beta parameter at index 1: {betas[1]}')
        if not 0.0 <= weight_decay:
            raise ValueError(f'Invalid weight_decay value: {weight_decay}')
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad, maximize=maximize)
        self.bias_correction = bias_correction
        self.exp_avg_dtype = exp_avg_dtype
        self.exp_avg_sq_dtype = exp_avg_sq_dtype
        self.use_adam = False
        super().__init__(params, defaults)

    def __setstate__(self, state):
        super().__setstate__(state)
        for group in self.param_groups:
            group.setdefault('amsgrad', False)
            group.setdefault('maximize', False)

    def _get_state_tensor(self, state, dtype):
        if dtype == torch.float32:
            return state
        if dtype not in (torch.uint8, torch.int8, torch.float16):
            raise TypeError(f'Unsupported dtype: {dtype}')
        return state.cast(Dtypes.dtype_to_qtype[dtype])

    @staticmethod
    def _update_lp_tensor(lp, hp):
        if lp is hp:
            return
        if isinstance(lp, ScalingTensor):
            lp.copy_(hp.cast(lp.qtype))
        else:
            lp.copy_(hp)

    def _new_state(self, p):
        shape_like = p.value if isinstance(p, ScalingTensor) else p
        z = torch.zeros(shape_like.shape, dtype=torch.float32, device=shape_like.device)
        return self._get_state_tensor(z, self.exp_avg_dtype), self._get_state_tensor(z.clone(), self.exp_avg_sq_dtype)

    @torch.no_grad()
    def lb_step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            if group['amsgrad']:
                raise ValueError('Only amsgrad=False is supported for now.')
            params, grads, ms, vs, steps = [], [], [], [], []
            beta1, beta2 = group['betas']
            for p in group['params']:
                g = p.grad
                if g is None:
                    continue
                if getattr(g, 'is_sparse', False):
                    raise RuntimeError('AdamW does not support sparse gradients')
                state = self.state[p]
                if len(state) == 0:
                    state['step'] = 0
                    state['exp_avg'], state['exp_avg_sq'] = self._new_state(p)
                state['step'] += 1
                params.append(p)
                grads.append(g)
                ms.append(state['exp_avg'])
                vs.append(state['exp_avg_sq'])
                steps.append(state['step'])
            self.adamw_fn(
                params, grads, ms, vs, [], steps, amsgrad=False, beta1=beta1, beta2=beta2, lr=group['lr'],
                weight_decay=group['weight_decay'], eps=group['eps'], maximize=group['maximize']
            )
        return loss

    def adamw_fn(self, params, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs, state_steps, *, amsgrad, beta1, beta2, lr, weight_decay,
                 eps, maximize):
        """One AdamW (or, with ``use_adam``, L2-regularised Adam) update over lists of tensors."""
        if amsgrad:
            raise ValueError('Only amsgrad=False is supported for now.')
        for i, p_lp in enumerate(params):
            g = grads[i].float()
            if maximize:
                g = -g
            p = p_lp.float()
            if p is p_lp or (not isinstance(p_lp, ScalingTensor) and p.data_ptr() == p_lp.data_ptr()):
                p = p.clone()
            if weight_decay != 0:
                if self.use_adam:
                    g = g.add(p, alpha=weight_decay)
                else:
                    p.mul_(1 - lr * weight_decay)
            m = exp_avgs[i].float()
            v = exp_avg_sqs[i].float()
            if m is exp_avgs[i]:
                m = m.clone()
            if v is exp_avg_sqs[i]:
                v = v.clone()
            step = state_steps[i]
            bc1 = 1 - beta1**step if self.bias_correction else 1.0
            bc2 = 1 - beta2**step if self.bias_correction else 1.0
            m.mul_(beta1).add_(g, alpha=1 - beta1)
            v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
            denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
            p.addcdiv_(m, denom, value=-lr / bc1)
            self._update_lp_tensor(p_lp, p)
            self._update_lp_tensor(exp_avgs[i], m)
            self._update_lp_tensor(exp_avg_sqs[i], v)
