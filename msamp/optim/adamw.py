"""LBAdamW (fused multi-tensor CUDA path) and FSDPAdamW.

On CUDA, one optimizer step is two launches over *all* parameters plus a tiny finalize kernel
(``csrc/optim.cu``), with the per-tensor scales of parameters and moments derived on the device.
On CPU the pure-torch definition of ``LBAdamWBase`` runs.  (reference: msamp/optim/adamw.py:19-337)
"""
import math

import torch
import torch.distributed as dist

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingMeta, ScalingTensor
from msamp.common.utils.dist import DistUtil
from msamp.optim.adamw_base import LBAdamWBase


class LBAdamW(LBAdamWBase):
    """AdamW with FP8 / FP16 optimizer states; ``tensor_scale=False`` stores the states unscaled."""
    def __init__(
        self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, amsgrad=False, *,
        maximize=False, exp_avg_dtype=torch.uint8, exp_avg_sq_dtype=torch.float16, tensor_scale=True
    ):
        self.tensor_scale = tensor_scale
        self._plans = {}
        # set by a sharded optimizer: fold the FP8 gradient reduce-scatter into stage 1 of the fused kernel
        # (dict(index={id(param): tensor index}, data_table, meta_table, world, rank, n_tensors)); consumed by one step
        self._reduce_in_step = None
        super().__init__(
            params, lr=lr, bias_correction=bias_correction, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=False,
            maximize=maximize, exp_avg_dtype=exp_avg_dtype, exp_avg_sq_dtype=exp_avg_sq_dtype
        )

    def adamw_fn(self, params, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs, state_steps, *, amsgrad, beta1, beta2, lr, weight_decay,
                 eps, maximize):
        if amsgrad:
            raise ValueError('Only amsgrad=False is supported for now.')
        if not params:
            return
        if not params[0].is_cuda:
            if self.tensor_scale:
                return super().adamw_fn(
                    params, grads, exp_avgs, exp_avg_sqs, max_exp_avg_sqs, state_steps, amsgrad=amsgrad, beta1=beta1, beta2=beta2,
                    lr=lr, weight_decay=weight_decay, eps=eps, maximize=maximize
                )
            raise NotImplementedError('tensor_scale=False is only implemented by the CUDA kernel')
        from msamp.ops.optim import FusedPlan
        entries = []
        for i, p in enumerate(params):
            step = state_steps[i]
            bc1 = 1 - beta1**step if self.bias_correction else 1.0
            bc2 = 1 - beta2**step if self.bias_correction else 1.0
            g = grads[i]
            if not isinstance(g, ScalingTensor) and not g.is_contiguous():
                g = g.contiguous()
            reduce = getattr(self, '_reduce_in_step', None)
            # A scaled-fp16 weight whose forward asked for an e4m3 copy (msamp.nn.functional.weight_fp8) gets that copy
            # from stage 2 of this kernel, which holds the new values anyway: the forward then finds it in its cache and the
            # separate re-quantisation pass over every weight (3 bytes per parameter and step) disappears.
            w8 = None
            if getattr(p, '_wants_fp8_copy', False) and isinstance(p, ScalingTensor) and p.meta.qtype == Dtypes.kfloat16 \
                    and p.value.dim() >= 2:
                w8 = getattr(p, '_adam_w8', None)
                if w8 is None or w8[0].numel() != p.numel() or w8[0].device != p.value.device:
                    w8 = p._adam_w8 = (torch.empty(p.numel(), dtype=torch.uint8, device=p.value.device),
                                       torch.empty((), dtype=torch.float32, device=p.value.device))
            entries.append(
                dict(
                    p=p, g=g, m=exp_avgs[i], v=exp_avg_sqs[i], w8=w8, g_index=(reduce['index'].get(id(p), -1) if reduce is not None else -1),
                    lr_wd_factor=(1.0 if self.use_adam else 1.0 - lr * weight_decay), l2=(weight_decay if self.use_adam else 0.0),
                    beta1=beta1, beta2=beta2, eps=eps, step_size=lr / bc1, sqrt_bc2=math.sqrt(bc2), gsign=(-1.0 if maximize else 1.0),
                    tensor_scale=self.tensor_scale
                )
            )
        key = (params[0].device, id(params[0]), len(params))
        plan = self._plans.get(key)
        if plan is None:
            plan = self._plans[key] = FusedPlan(params[0].device)
        plan.run(entries, reduce=getattr(self, '_reduce_in_step', None))
        for e in entries:
            if e['w8'] is not None:
                p, (w8, sinv) = e['p'], e['w8']
                val = p.value
                key = (val.data_ptr(), val._version, p.meta.scale_inv._version, p.meta.scale_inv.data_ptr())
                p._fp8_cache1 = (key, w8.view(-1, val.shape[-1]), sinv)

    def __getstate__(self):
        d = super().__getstate__() if hasattr(super(), '__getstate__') else self.__dict__.copy()
        d = dict(d)
        d['_plans'] = {}
        d['_reduce_in_step'] = None
        return d


class FSDPAdamW(LBAdamWBase):
    """AdamW for FSDP flat parameters that carry FP8 weight bytes.

    Each sharded FP8 parameter (an fp32-viewed slice with a ``_meta``) gets a scaled-fp16 master copy;
    ``param.grad`` bytes are wrapped as an FP8 ScalingTensor using ``_grad_meta``; after the update
    the master is re-quantised into the shard with an amax that is MAX-reduced over all shards,
    because a tensor's scale is global while its bytes are sharded.
    """
    def __init__(
        self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, amsgrad=False, *,
        maximize=False, exp_avg_dtype=torch.uint8, exp_avg_sq_dtype=torch.float16, tensor_scale=True
    ):
        self.tensor_scale = tensor_scale
        super().__init__(
            params, lr=lr, bias_correction=bias_correction, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=False,
            maximize=maximize, exp_avg_dtype=exp_avg_dtype, exp_avg_sq_dtype=exp_avg_sq_dtype
        )
        self.original_params = []
        self.master_weights = []
        for group in self.param_groups:
            new_params = []
            for param in group['params']:
                if param is None:
                    continue
                self.original_params.append(param)
                meta = getattr(param, '_meta', None)
                if meta is not None and param.numel() > 0:
                    payload = ScalingTensor(param.detach().view(Dtypes.get_dtype_from_qtype(meta.qtype)), meta)
                    master = payload.cast(Dtypes.kfloat16)
                    master.requires_grad = True
                    self.master_weights.append(master)
                    new_params.append(master)
                else:
                    self.master_weights.append(None)
                    new_params.append(param)
            group['params'] = new_params

    def zero_grad(self, set_to_none=False):
        for p in self.original_params:
            if p.grad is None:
                continue
            if set_to_none:
                p.grad = None
            else:
                p.grad.detach_()
                p.grad.requires_grad_(False)
                p.grad.zero_()

    def step(self, closure=None):
        for master, p in zip(self.master_weights, self.original_params):
            if master is not None and p.grad is not None:
                gmeta = p._grad_meta
                master.grad = ScalingTensor(p.grad.view(Dtypes.get_dtype_from_qtype(gmeta.qtype)), gmeta)
                p.grad = None
        rtn = super().step(closure)
        world = DistUtil.get_world_size()
        for master, p in zip(self.master_weights, self.original_params):
            meta = getattr(p, '_meta', None)
            if meta is None:
                continue
            hp = None
            if master is None or p.numel() == 0:
                meta.amax[0].zero_()
            else:
                hp = master.float()
                meta.amax[0] = hp.abs().max()
            if world > 1:
                dist.all_reduce(meta.amax[0], op=dist.ReduceOp.MAX)
            meta.reset_scaling_factor()
            if hp is not None:
                with ScalingMeta.in_time_scaling_context(False):
                    q = hp.cast(meta.qtype, meta, False)
                p.data.copy_(q.value.view(p.dtype).view_as(p))
            else:
                meta.scale_inv.copy_(torch.reciprocal(meta.scale))
        return rtn
