"""Base class of the low-bit optimizers.

``step`` = ``lb_step`` (the parameter update, implemented by subclasses) followed by the
delayed-scaling bookkeeping for every FP8Linear registered in ``model_state``.  ``state_dict`` /
``load_state_dict`` accept ScalingTensor parameters and states and never change the dtype of a
saved state.  (reference: msamp/optim/optimizer.py:20-284)
"""
import warnings
from collections import defaultdict
from collections.abc import Iterable
from copy import deepcopy
from itertools import chain

import torch
from torch.optim.optimizer import Optimizer, required

from msamp.common.tensor import ScalingMeta, ScalingTensor, TensorDist
from msamp.nn import ScalingParameter, model_state
from msamp.ops import cast as _k


class LBOptimizer(Optimizer):
    """Optimizer base that understands ScalingTensor parameters, gradients and states."""
    def __init__(self, params, defaults):
        super().__init__(params, defaults)
        self.set_grad_none = False

    def step(self, closure=None):
        rtn = self.lb_step(closure)
        self._update_scaling_factors()
        return rtn

    def lb_step(self, closure=None):
        raise NotImplementedError('lb_step is not implemented')

    def all_reduce_grads(self, model):
        """Average the FP8 weight gradients over the default group (a no-op when FP8 DDP already did it)."""
        if model_state.use_fp8_ddp:
            return
        grads = [p.grad for p in model.parameters() if isinstance(p, ScalingParameter) and p.grad is not None]
        TensorDist.all_reduce_avg(grads)

    def _update_scaling_factors(self, training=True):
        """Roll the amax windows of all registered layers and refresh their delayed scales (one launch per kind)."""
        if not model_state.ready_to_scale_tensor:
            return
        model_state.ready_to_scale_tensor = False
        metas = model_state.flattened_scaling_metas
        if metas is None:
            return
        names = ['input']
        if training:
            names.append('ograd')
            if not ScalingMeta.in_time_scaling:
                names.append('wgrad')
        for name in names:
            flat = metas[name]
            self._apply_pending_resets(flat)
            bad = flat.get('_bad_dev')
            if bad is None or bad.device != flat['amaxs'].device or bad.numel() != flat['amaxs'].shape[0]:
                bad = flat['_bad_dev'] = torch.zeros(flat['amaxs'].shape[0], dtype=torch.int32, device=flat['amaxs'].device)
            _k.roll_windows(flat['amaxs'], flat['scales'], flat['qtype'], margin=0, bad_out=bad)
            flat['amax_counters'] += 1
            # A non-finite amax puts its meta back into warm-up (in-time scaling for `window` steps), as the reference does
            # (msamp/optim/optimizer.py:100-103).  The step counters live on the host, the flags on the device: on CPU the
            # reset is immediate; on CUDA the flags travel through pinned memory and are applied once their copy has
            # finished (at the latest before the next roll), so that no step waits for the device.
            if bad.is_cuda:
                host = flat.get('_bad_host')
                if host is None or host.numel() != bad.numel():
                    host = flat['_bad_host'] = torch.zeros(bad.numel(), dtype=torch.int32).pin_memory()
                host.copy_(bad, non_blocking=True)
                event = torch.cuda.Event()
                event.record()
                flat['_bad_pending'] = (host, event)
            else:
                flat['_bad_pending'] = (bad.clone(), None)
                self._apply_pending_resets(flat)

    @staticmethod
    def _apply_pending_resets(flat, wait=True):
        pending = flat.get('_bad_pending')
        if pending is None:
            return
        host, event = pending
        if event is not None:
            if not wait and not event.query():
                return
            event.synchronize()    # the copy was enqueued a whole step ago: this does not stall in practice
        mask = host.bool()
        if bool(mask.any()):
            flat['amax_counters'][mask.to(flat['amax_counters'].device)] = 0
        flat['_bad_pending'] = None

    # ---- bookkeeping that must tolerate ScalingTensor --------------------------------------------
    def zero_grad(self, set_to_none=None):
        if set_to_none is None:
            set_to_none = self.set_grad_none
        for group in self.param_groups:
            for p in group['params']:
                if p.grad is None:
                    continue
                if set_to_none:
                    p.grad = None
                elif isinstance(p.grad, ScalingTensor):
                    p.grad.zero_()
                else:
                    p.grad.detach_()
                    p.grad.requires_grad_(False)
                    p.grad.zero_()

    def state_dict(self):
        """``{'state': {index: {...}}, 'param_groups': [...]}`` with parameters replaced by their order index."""
        mapping = {}
        start = 0

        def pack(group):
            nonlocal start
            packed = {k: v for k, v in group.items() if k != 'params'}
            mapping.update({id(p): i for i, p in enumerate(group['params'], start) if id(p) not in mapping})
            packed['params'] = [mapping[id(p)] for p in group['params']]
            start += len(packed['params'])
            return packed

        groups = [pack(g) for g in self.param_groups]
        state = {(mapping[id(k)] if isinstance(k, (torch.Tensor, ScalingTensor)) else k): v for k, v in self.state.items()}
        return {'state': state, 'param_groups': groups}

    def load_state_dict(self, state_dict):
        state_dict = deepcopy(state_dict)
        groups, saved = self.param_groups, state_dict['param_groups']
        if len(groups) != len(saved):
            raise ValueError('loaded state dict has a different number of parameter groups')
        if any(len(g['params']) != len(s['params']) for g, s in zip(groups, saved)):
            raise ValueError("loaded state dict contains a parameter group that doesn't match the size of optimizer's group")
        id_map = dict(zip(chain.from_iterable(g['params'] for g in saved), chain.from_iterable(g['params'] for g in groups)))

        def move(param, value, key=None):
            if isinstance(value, torch.Tensor):
                return value if key == 'step' else value.to(param.device)
            if isinstance(value, ScalingTensor):
                return value.to(device=param.device)
            if isinstance(value, dict):
                return {k: move(param, v, key=k) for k, v in value.items()}
            if isinstance(value, Iterable) and not isinstance(value, (str, bytes)):
                return type(value)(move(param, v) for v in value)
            return value

        state = defaultdict(dict)
        for k, v in state_dict['state'].items():
            if k in id_map:
                state[id_map[k]] = move(id_map[k], v)
            else:
                state[k] = v
        new_groups = []
        for g, s in zip(groups, saved):
            s['params'] = g['params']
            new_groups.append(s)
        self.__setstate__({'state': state, 'param_groups': new_groups})

    def add_param_group(self, param_group):
        if not isinstance(param_group, dict):
            raise TypeError('param group must be a dict')
        params = param_group['params']
        if isinstance(params, (torch.Tensor, ScalingTensor)):
            param_group['params'] = [params]
        elif isinstance(params, set):
            raise TypeError('optimizer parameters need to be organized in ordered collections; please use a list instead of a set.')
        else:
            param_group['params'] = list(params)
        for p in param_group['params']:
            if not isinstance(p, (torch.Tensor, ScalingTensor)):
                raise TypeError('optimizer can only optimize Tensors, but one of the params is ' + torch.typename(p))
            if not self.defaults.get('differentiable', None) and not (p.is_leaf or p.retains_grad):
                raise ValueError("can't optimize a non-leaf Tensor")
        for name, default in self.defaults.items():
            if default is required and name not in param_group:
                raise ValueError(f"parameter group didn't specify a value of required optimization parameter {name}")
            param_group.setdefault(name, default)
        ids = [id(p) for p in param_group['params']]
        if len(ids) != len(set(ids)):
            warnings.warn('optimizer contains a parameter group with duplicate parameters', stacklevel=3)
        seen = set(id(p) for g in self.param_groups for p in g['params'])
        if not seen.isdisjoint(ids):
            raise ValueError('some parameters appear in more than one parameter group')
        self.param_groups.append(param_group)
