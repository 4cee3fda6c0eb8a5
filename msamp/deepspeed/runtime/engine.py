"""MSAMPDeepSpeedEngine: the DeepSpeed training-engine surface on msamp's optimizers and collectives.

Mirrors what the reference's engine does on top of DeepSpeed (msamp/deepspeed/runtime/engine.py:61-486):
build the basic optimizer from the config, run ``msamp.initialize`` (``O3`` converts like ``O2`` and then
shards with FP8 weights), pick ``FP8Optimizer`` (no ZeRO) or ``FP8DeepSpeedZeroOptimizer`` (ZeRO 1/2), scale
the loss by the accumulation steps, step at accumulation boundaries, and save/load checkpoints.
"""
import os

import torch
import torch.distributed as dist

import msamp
from msamp.common.utils import logger
from msamp.common.utils.dist import DistUtil
from msamp.deepspeed.runtime.fp8.fused_optimizer import FP8Optimizer
from msamp.deepspeed.runtime.zero.fp8_stage_1_and_2 import FP8DeepSpeedZeroOptimizer
from msamp.utils.metrics import StepMetrics
from msamp.utils.timer import PhaseTimers, nvtx_range

_OPTIMIZERS = {'adam': torch.optim.Adam, 'adamw': torch.optim.AdamW}


def build_over_all_parameters(build, model_parameters, module):
    """Basic (torch) optimizer over ``model_parameters`` or all parameters of ``module``.

    Models built from ``msamp.te`` modules already hold ScalingParameters, which torch's optimizers reject: the optimizer
    is then built on the plain tensors and its first group rebound to the full list (``msamp.initialize`` replaces every
    entry by position anyway)."""
    params = list(model_parameters) if model_parameters is not None else list(module.parameters())
    if params and isinstance(params[0], dict):
        return build(params)
    plain = [p for p in params if torch.is_tensor(p)]
    if len(plain) == len(params):
        return build(params)
    opt = build(plain if plain else [torch.nn.Parameter(torch.zeros(1))])
    opt.param_groups[0]['params'] = params
    return opt


class _WarmupLR:
    """Linear warm-up from ``warmup_min_lr`` to ``warmup_max_lr`` over ``warmup_num_steps`` (DeepSpeed's WarmupLR)."""
    def __init__(self, optimizer, warmup_min_lr=0.0, warmup_max_lr=1e-3, warmup_num_steps=1000, **unused):
        self.optimizer, self.lo, self.hi, self.n = optimizer, warmup_min_lr, warmup_max_lr, max(1, warmup_num_steps)
        self.last_step = 0
        self._apply()

    def _apply(self):
        frac = min(1.0, self.last_step / self.n)
        for g in self.optimizer.param_groups:
            g['lr'] = self.lo + (self.hi - self.lo) * frac

    def step(self):
        self.last_step += 1
        self._apply()

    def get_lr(self):
        return [g['lr'] for g in self.optimizer.param_groups]

    def state_dict(self):
        return {'last_step': self.last_step}

    def load_state_dict(self, sd):
        self.last_step = sd['last_step']
        self._apply()


class MSAMPDeepSpeedEngine(torch.nn.Module):
    """Training engine: ``loss = engine(batch); engine.backward(loss); engine.step()``."""
    def __init__(self, args=None, model=None, optimizer=None, model_parameters=None, training_data=None, lr_scheduler=None, mpu=None,
                 collate_fn=None, config=None):
        super().__init__()
        self.config = config
        self.mpu = mpu
        self.dp_group = mpu.get_data_parallel_group() if mpu is not None and hasattr(mpu, 'get_data_parallel_group') else None
        self.dp_world_size = DistUtil.get_world_size(self.dp_group)
        self.global_rank = DistUtil.get_rank()
        self.timers = PhaseTimers(enabled=config.wall_clock_breakdown)
        self.metrics = StepMetrics(rank=self.global_rank)
        self.micro_steps = 0
        self.global_steps = 0
        self.skipped_steps = 0
        self.global_samples = 0
        self.module = model
        self._configure_optimizer(optimizer, model_parameters)
        self.lr_scheduler = self._configure_scheduler(lr_scheduler)
        self.training_dataloader = self._configure_dataloader(training_data, collate_fn)

    # ------------------------------------------------------------------ configuration
    def _configure_basic_optimizer(self, model_parameters):
        name = (self.config.optimizer_name or 'adamw').lower()
        if name not in _OPTIMIZERS:
            raise ValueError(f'optimizer {name} is not supported with msamp (use Adam or AdamW)')
        params = dict(self.config.optimizer_params)
        params.pop('torch_adam', None)
        adam_w_mode = params.pop('adam_w_mode', name == 'adamw')
        cls = torch.optim.AdamW if adam_w_mode else torch.optim.Adam
        return build_over_all_parameters(lambda ps: cls(ps, **params), model_parameters, self.module)

    def _configure_optimizer(self, client_optimizer, model_parameters):
        cfg = self.config
        basic = client_optimizer if client_optimizer is not None and not callable(client_optimizer) else None
        if basic is None:
            basic = client_optimizer(model_parameters) if callable(client_optimizer) else self._configure_basic_optimizer(model_parameters)
        self.basic_optimizer = basic
        if not cfg.msamp_enabled:
            self.optimizer = basic
            self._plain = True
            return
        self._plain = False
        level = cfg.msamp_optlevel
        init_level = 'O2' if level == 'O3' else level    # sharding below provides the FP8 weights + fp16 masters of O3
        src = dist.get_global_rank(self.dp_group, 0) if (self.dp_group is not None and dist.is_initialized()) else 0
        self.module, lb_opt = msamp.initialize(self.module, basic, init_level, use_te=bool(cfg.msamp_use_te), group=self.dp_group, src_rank=src)
        dyn_args = dict(init_scale=2**cfg.initial_scale_power, scale_window=cfg.loss_scale_window, min_scale=cfg.min_loss_scale,
                        delayed_shift=cfg.hysteresis)
        dynamic = cfg.fp16_enabled and cfg.loss_scale == 0
        static = cfg.loss_scale if (cfg.fp16_enabled and cfg.loss_scale > 0) else 1.0
        if cfg.zero_enabled:
            if cfg.zero_optimization_stage > 2:
                raise NotImplementedError('ZeRO stage 3 with FP8 is provided by msamp.fsdp.FP8FullyShardedDataParallel')
            self.optimizer = FP8DeepSpeedZeroOptimizer(
                self.module, lb_opt, static_loss_scale=static, dynamic_loss_scale=dynamic, dynamic_loss_args=dyn_args,
                clip_grad=cfg.gradient_clipping, dp_process_group=self.dp_group, partition_grads=cfg.zero_optimization_stage == 2,
                mpu=self.mpu, timers=self.timers, reduce_bucket_size=cfg.zero_reduce_bucket_size, overlap_comm=cfg.zero_overlap_comm
            )
        else:
            self.optimizer = FP8Optimizer(
                self.module, lb_opt, static_loss_scale=static, dynamic_loss_scale=dynamic, dynamic_loss_args=dyn_args,
                clip_grad=cfg.gradient_clipping, fp8_master=(level == 'O3'), zero_stage=0, group=self.dp_group, mpu=self.mpu,
                timers=self.timers
            )
            if self.optimizer.zero is None and self.dp_world_size > 1:
                # replicated states: FP8 all-reduce of weight gradients through the sharded-optimizer machinery at stage 0
                from msamp.parallel.zero import ZeroShardedOptimizer
                self.optimizer.zero = ZeroShardedOptimizer(self.module, lb_opt, stage=0, group=self.dp_group)

    def _configure_scheduler(self, client):
        if client is not None:
            return client(self.basic_optimizer) if callable(client) and not hasattr(client, 'step') else client
        if self.config.scheduler_name:
            if self.config.scheduler_name != 'WarmupLR':
                raise ValueError(f'scheduler {self.config.scheduler_name} is not built in; pass an lr_scheduler object')
            target = self.optimizer if hasattr(self.optimizer, 'param_groups') else self.basic_optimizer
            return _WarmupLR(target, **self.config.scheduler_params)
        return None

    def _configure_dataloader(self, data, collate_fn):
        if data is None:
            return None
        sampler = None
        if self.dp_world_size > 1:
            sampler = torch.utils.data.distributed.DistributedSampler(data, num_replicas=self.dp_world_size, rank=DistUtil.get_rank(self.dp_group))
        return torch.utils.data.DataLoader(data, batch_size=self.config.train_micro_batch_size_per_gpu, sampler=sampler, collate_fn=collate_fn,
                                           shuffle=sampler is None)

    # ------------------------------------------------------------------ properties
    def gradient_accumulation_steps(self):
        return self.config.gradient_accumulation_steps

    def train_micro_batch_size_per_gpu(self):
        return self.config.train_micro_batch_size_per_gpu

    def train_batch_size(self):
        return self.config.train_batch_size

    def is_gradient_accumulation_boundary(self):
        return (self.micro_steps + 1) % self.gradient_accumulation_steps() == 0

    def get_lr(self):
        groups = self.optimizer.param_groups if hasattr(self.optimizer, 'param_groups') else self.basic_optimizer.param_groups
        return [g['lr'] for g in groups]

    # ------------------------------------------------------------------ training loop
    def forward(self, *inputs, **kwargs):
        with nvtx_range('forward'), self.timers.phase('forward'):
            return self.module(*inputs, **kwargs)

    def backward(self, loss, retain_graph=False):
        with nvtx_range('backward'), self.timers.phase('backward'):
            ga = self.gradient_accumulation_steps()
            if ga > 1:
                loss = loss / ga
            if self._plain:
                loss.backward(retain_graph=retain_graph)
            else:
                self.optimizer.backward(loss, retain_graph=retain_graph)
        return loss

    def allreduce_gradients(self, bucket_size=None):
        """Average high-precision gradients when no sharded optimizer does it (plain torch optimizer, several ranks)."""
        if self.dp_world_size == 1:
            return
        for p in self.module.parameters():
            if torch.is_tensor(p) and p.grad is not None:
                dist.all_reduce(p.grad, group=self.dp_group)
                p.grad.div_(self.dp_world_size)

    def step(self):
        boundary = self.is_gradient_accumulation_boundary()
        if boundary:
            with nvtx_range('step'), self.timers.phase('step'):
                if self._plain:
                    self.allreduce_gradients()
                    if self.config.gradient_clipping > 0:
                        self._clip_plain(self.config.gradient_clipping)
                    self.optimizer.step()
                    self.optimizer.zero_grad(set_to_none=True)
                    skipped = False
                else:
                    skipped = self.optimizer.step()
                    self.optimizer.zero_grad(set_to_none=True)
            if skipped:
                self.skipped_steps += 1
                self.metrics.skipped_steps += 1
            elif self.lr_scheduler is not None:
                self.lr_scheduler.step()
            self.global_steps += 1
            self.global_samples += self.train_batch_size()
            if self.config.wall_clock_breakdown and self.global_steps % self.config.steps_per_print == 0 and self.global_rank == 0:
                logger.info(f'step {self.global_steps}: ' + self.timers.log(reset=True))
        self.micro_steps += 1

    def _clip_plain(self, max_norm):
        """Global-norm clipping without FP8 gradients; the norm is summed over the model-parallel group if there is one."""
        grads = [p.grad for p in self.module.parameters() if p.grad is not None]
        if not grads:
            return
        sq = torch.stack([g.detach().float().pow(2).sum() for g in grads]).sum().reshape(1)
        mp_group = self.mpu.get_model_parallel_group() if (self.mpu is not None and hasattr(self.mpu, 'get_model_parallel_group')) else None
        if mp_group is not None and dist.is_initialized() and dist.get_world_size(mp_group) > 1:
            dist.all_reduce(sq, group=mp_group)
        coef = torch.clamp(max_norm / (sq.sqrt()[0] + 1e-6), max=1.0)
        for g in grads:
            g.mul_(coef.to(g.dtype))

    def train_batch(self, data_iter):
        """Convenience: one full batch (all accumulation steps) from an iterator of ``(inputs, labels)``-like tuples."""
        total = 0.0
        for _ in range(self.gradient_accumulation_steps()):
            batch = next(data_iter)
            loss = self(*batch) if isinstance(batch, (tuple, list)) else self(batch)
            self.backward(loss)
            self.step()
            total += float(loss.detach())
        return total / self.gradient_accumulation_steps()

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, save_dir, tag=None, client_state=None):
        tag = tag or f'global_step{self.global_steps}'
        path = os.path.join(save_dir, str(tag))
        os.makedirs(path, exist_ok=True)
        if DistUtil.get_rank(self.dp_group) == 0:
            torch.save({'module': self.module.state_dict(), 'global_steps': self.global_steps, 'global_samples': self.global_samples,
                        'skipped_steps': self.skipped_steps, 'lr_scheduler': self.lr_scheduler.state_dict() if self.lr_scheduler else None,
                        'client_state': client_state or {}}, os.path.join(path, 'mp_rank_00_model_states.pt'))
            with open(os.path.join(save_dir, 'latest'), 'w') as f:
                f.write(str(tag))
        rank = DistUtil.get_rank(self.dp_group)
        torch.save({'optimizer_state_dict': self.optimizer.state_dict()}, os.path.join(path, f'zero_pp_rank_{rank}_mp_rank_00_optim_states.pt'))
        if dist.is_initialized() and self.dp_world_size > 1:
            dist.barrier(group=self.dp_group)
        return True

    def load_checkpoint(self, load_dir, tag=None, load_optimizer_states=True, load_lr_scheduler_states=True):
        if tag is None:
            with open(os.path.join(load_dir, 'latest')) as f:
                tag = f.read().strip()
        path = os.path.join(load_dir, str(tag))
        states = torch.load(os.path.join(path, 'mp_rank_00_model_states.pt'), map_location='cpu', weights_only=False)
        self.module.load_state_dict(states['module'])
        self.global_steps, self.global_samples, self.skipped_steps = states['global_steps'], states['global_samples'], states['skipped_steps']
        if load_lr_scheduler_states and self.lr_scheduler is not None and states.get('lr_scheduler'):
            self.lr_scheduler.load_state_dict(states['lr_scheduler'])
        if load_optimizer_states:
            rank = DistUtil.get_rank(self.dp_group)
            opt = torch.load(os.path.join(path, f'zero_pp_rank_{rank}_mp_rank_00_optim_states.pt'), map_location='cpu', weights_only=False)
            self.optimizer.load_state_dict(opt['optimizer_state_dict'])
        return path, states.get('client_state', {})
