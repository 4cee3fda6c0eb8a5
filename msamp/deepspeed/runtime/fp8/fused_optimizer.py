"""FP8Optimizer: loss scaling, overflow skipping, clipping and master weights around a low-bit optimizer.

Semantics of the reference's DeepSpeed fused-optimizer analogue (msamp/deepspeed/runtime/fp8/fused_optimizer.py:23-618):
FP8 parameters keep scaled-fp16 masters and e4m3 model weights, the step is skipped and the loss scale
reduced when any gradient overflowed, gradients are unscaled and clipped through ``scale_inv`` for
ScalingTensors, and the checkpoint uses the keys ``dynamic_loss_scale, cur_scale, cur_iter,
last_overflow_iter, scale_factor, scale_window, optimizer_state_dict, fp32_groups_flat, fp8_master_groups, clip_grad``.
"""
import torch

from msamp.common.tensor import ScalingTensor
from msamp.deepspeed.runtime.fp8.loss_scaler import DynamicLossScaler, LossScaler
from msamp.deepspeed.runtime.utils import MSAMPCheckOverflow
from msamp.parallel.zero import ZeroShardedOptimizer
from msamp.utils.timer import PhaseTimers

OVERFLOW_CHECK, COMPUTE_NORM, UNSCALE_AND_CLIP, BASIC_STEP, UPDATE_FP16 = (
    'overflow_check', 'compute_norm', 'unscale_and_clip', 'basic_step', 'update_fp16'
)


class FP8Optimizer:
    """Wraps ``init_optimizer`` (an LB optimizer) for a model converted by ``msamp.initialize``."""
    def __init__(self, model, init_optimizer, static_loss_scale=1.0, dynamic_loss_scale=False, initial_dynamic_scale=2**32,
                 dynamic_loss_args=None, clip_grad=0.0, fp8_master=True, zero_stage=0, group=None, mpu=None, timers=None):
        self.model, self.optimizer, self.clip_grad = model, init_optimizer, clip_grad
        self.mpu = mpu
        self.timers = timers or PhaseTimers(enabled=False)
        if dynamic_loss_scale:
            args = dict(dynamic_loss_args or {})
            self.loss_scaler = DynamicLossScaler(
                init_scale=args.get('init_scale', initial_dynamic_scale), scale_window=args.get('scale_window', 1000),
                min_scale=args.get('min_scale', 1.0), hysteresis=args.get('delayed_shift', 2)
            )
        else:
            self.loss_scaler = LossScaler(static_loss_scale)
        self.dynamic_loss_scale = dynamic_loss_scale
        stage = zero_stage if zero_stage else (1 if fp8_master else 0)
        self.zero = ZeroShardedOptimizer(model, init_optimizer, stage=stage, group=group) if (fp8_master or zero_stage) else None
        self.overflow_checker = MSAMPCheckOverflow(group=group, mpu=mpu)
        self.overflow = False
        self.skipped_steps = 0
        self._global_grad_norm = 0.0

    @property
    def cur_scale(self):
        return self.loss_scaler.cur_scale

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    @property
    def state(self):
        return self.optimizer.state

    def _all_params(self):
        if self.zero is not None:
            return list(self.zero.fp8_params) + list(self.zero.hp_params) + list(self.zero.local_params)
        return [p for g in self.optimizer.param_groups for p in g['params']]

    def zero_grad(self, set_to_none=True):
        for p in self._all_params():
            if p.grad is None:
                continue
            if set_to_none or isinstance(p.grad, ScalingTensor):
                p.grad = None
            else:
                p.grad.zero_()
        if self.zero is not None:
            # parameters this rank does not own are not in the inner optimizer, but their gradients exist here too
            for p in self.zero.fp8_params:
                p.grad = None
            if self.zero.hp_layout:
                self.zero._clear_hp_grads()

    def backward(self, loss, retain_graph=False):
        """Scale the loss and back-propagate."""
        (loss.float() * self.cur_scale).backward(retain_graph=retain_graph)

    def _unscale_and_clip(self, params, sharded=()):
        """Unscale and clip the gradients of ``params`` (held by every rank) and of ``sharded`` (each held by one rank
        of the data-parallel group only: their squared norms are summed over the group so that all ranks clip alike)."""
        sharded = list(sharded)
        grads = [p.grad for p in list(params) + sharded if p.grad is not None]
        with self.timers.phase(COMPUTE_NORM):
            from msamp.nn.clip_grad import _grad_norm

            def sumsq(ps):
                acc = None
                for p in ps:
                    if p.grad is not None:
                        n = _grad_norm(p.grad, 2.0)**2
                        acc = n if acc is None else acc + n.to(acc.device)
                return acc

            sq = sumsq(params)
            if self.zero is not None and self.zero.world > 1 and (self.zero.sharded or sharded):
                part = sumsq(sharded)
                part = part if part is not None else torch.zeros((), device=self.zero.device)
                part = part.float().reshape(1).clone()
                torch.distributed.all_reduce(part, group=self.zero.group)
                sq = part[0] if sq is None else sq + part[0].to(sq.device)
            else:
                part = sumsq(sharded)
                if part is not None:
                    sq = part if sq is None else sq + part.to(sq.device)
            mp_group = self.mpu.get_model_parallel_group() if (self.mpu is not None and hasattr(self.mpu, 'get_model_parallel_group')) else None
            if mp_group is not None and torch.distributed.get_world_size(mp_group) > 1:
                # pipeline stages / tensor-parallel ranks hold different parameters of one model: one global norm
                part = (sq if sq is not None else torch.zeros(())).float().reshape(1).clone()
                torch.distributed.all_reduce(part, group=mp_group)
                sq = part[0]
            total = (sq.sqrt() / self.cur_scale) if sq is not None else torch.zeros(())
        with self.timers.phase(UNSCALE_AND_CLIP):
            combined = self.cur_scale
            if self.clip_grad > 0:
                clip = (total / self.clip_grad).clamp(min=1.0)
                combined = clip * self.cur_scale
            if not (isinstance(combined, float) and combined == 1.0):
                for g in grads:
                    if isinstance(g, ScalingTensor):
                        g.div_(combined)
                    else:
                        g.div_(combined if isinstance(combined, float) else combined.to(g.device, g.dtype))
        self._global_grad_norm = total
        return total

    def step(self, closure=None):
        """One optimizer step; returns True when the step was skipped because of an overflow."""
        params = self._all_params()
        with self.timers.phase(OVERFLOW_CHECK):
            self.overflow = self.overflow_checker.check(params) if (self.dynamic_loss_scale or self.cur_scale != 1.0) else False
        prev = self.cur_scale
        self.loss_scaler.update_scale(self.overflow)
        if self.overflow:
            self.skipped_steps += 1
            from msamp.common.utils import logger
            logger.info(f'[msamp] OVERFLOW! Skipping step. Attempted loss scale: {prev}, reducing to {self.cur_scale}')
            self.zero_grad()
            return True
        if self.zero is not None:
            # gradient exchange first (no-op for one rank), then unscale/clip on what this rank will update
            self.zero._reduce_fp8_grads()
            self.zero._reduce_hp_grads()
            if self.zero.sharded:
                for i, m in self.zero.masters.items():
                    m.grad = self.zero.fp8_params[i].grad
                if self.zero.world > 1:
                    # high-precision parameters are sharded as well: each rank unscales and clips what it owns
                    self._unscale_and_clip([], sharded=list(self.zero.masters.values()) + self.zero._owned_hp() + self.zero.local_params)
                else:
                    self._unscale_and_clip(self.zero.hp_params, sharded=list(self.zero.masters.values()) + self.zero.local_params)
            else:
                local = {id(p) for p in self.zero.local_params}
                self._unscale_and_clip([p for p in params if id(p) not in local], sharded=self.zero.local_params)
            with self.timers.phase(BASIC_STEP):
                self.optimizer.step()
            with self.timers.phase(UPDATE_FP16):
                if self.zero.sharded:
                    self.zero._publish_weights()
                    self.zero._gather_hp_params()
                    for m in self.zero.masters.values():
                        m.grad = None
            for p in self.zero.fp8_params:
                p.grad = None
            if self.zero.hp_layout:
                self.zero._clear_hp_grads()
        else:
            self._unscale_and_clip(params)
            with self.timers.phase(BASIC_STEP):
                self.optimizer.step()
        return False

    def get_global_grad_norm(self):
        return self._global_grad_norm

    def state_dict(self):
        sd = {'dynamic_loss_scale': self.dynamic_loss_scale, 'cur_scale': self.cur_scale, 'cur_iter': getattr(self.loss_scaler, 'cur_iter', 0)}
        if self.dynamic_loss_scale:
            sd.update(last_overflow_iter=self.loss_scaler.last_overflow_iter, scale_factor=self.loss_scaler.scale_factor,
                      scale_window=self.loss_scaler.scale_window)
        sd['optimizer_state_dict'] = self.optimizer.state_dict()
        hp = self.zero.hp_params if self.zero is not None else [p for p in self._all_params() if not isinstance(p, ScalingTensor)]
        sd['fp32_groups_flat'] = [torch.cat([p.detach().float().reshape(-1) for p in hp])] if hp else []
        sd['fp8_master_groups'] = [[m.detach() for m in g] for g in self.zero._master_groups()] if (self.zero and self.zero.sharded) else []
        sd['clip_grad'] = self.clip_grad
        return sd

    def load_state_dict(self, sd, load_optimizer_states=True):
        self.dynamic_loss_scale = sd['dynamic_loss_scale']
        self.loss_scaler.cur_scale = sd['cur_scale']
        if self.dynamic_loss_scale:
            self.loss_scaler.cur_iter = sd['cur_iter']
            self.loss_scaler.last_overflow_iter = sd['last_overflow_iter']
            self.loss_scaler.scale_factor = sd['scale_factor']
            self.loss_scaler.scale_window = sd['scale_window']
        if load_optimizer_states:
            self.optimizer.load_state_dict(sd['optimizer_state_dict'])
        self.clip_grad = sd['clip_grad']
        hp = self.zero.hp_params if self.zero is not None else [p for p in self._all_params() if not isinstance(p, ScalingTensor)]
        if sd['fp32_groups_flat']:
            flat, off = sd['fp32_groups_flat'][0], 0
            for p in hp:
                p.data.copy_(flat[off:off + p.numel()].view_as(p).to(p.dtype))
                off += p.numel()
        if sd['fp8_master_groups'] and self.zero is not None and self.zero.sharded:
            groups, saved = self.zero._master_groups(), sd['fp8_master_groups']
            if len(saved) == 1 and len(groups) != 1 and len(saved[0]) == sum(len(g) for g in groups):
                # files written before the per-group nesting: one list in ascending tensor index
                pairs = list(zip([self.zero.masters[i] for i in sorted(self.zero.masters)], saved[0]))
            else:
                if len(saved) != len(groups) or any(len(a) != len(b) for a, b in zip(saved, groups)):
                    raise ValueError('fp8 master groups of the checkpoint do not match the optimizer\'s parameter groups')
                pairs = [(m, t) for gm, gt in zip(groups, saved) for m, t in zip(gm, gt)]
            for master, tensor in pairs:
                master.copy_(tensor.to(device=self.zero.device))
            self.zero._publish_weights()
