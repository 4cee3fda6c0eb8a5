"""Engine with DeepSpeed's constructor flow, hook names and training-loop calls (nothing more)."""
import torch


class _Timers:
    def __call__(self, name):
        return self

    def start(self):
        pass

    def stop(self):
        pass


class DeepSpeedEngine(torch.nn.Module):
    def __init__(self, args, model, optimizer=None, model_parameters=None, training_data=None, lr_scheduler=None, mpu=None,
                 dist_init_required=None, collate_fn=None, config=None, config_class=None, dont_change_device=False):
        super().__init__()
        self.mpu = mpu
        self._config = config_class
        self.module = model
        self.timers = _Timers()
        self.micro_steps = 0
        self.global_steps = 0
        self.skipped_steps = 0
        self.training_dataloader = None
        self.optimizer = None
        self.basic_optimizer = None
        self.lr_scheduler = None
        self._configure_optimizer(optimizer, model_parameters)
        self._configure_lr_scheduler(lr_scheduler)

    # ---- config accessors (DeepSpeed exposes its config through methods of the engine)
    def fp16_enabled(self):
        return self._config.fp16_enabled

    def dynamic_loss_scale(self):
        return self._config.loss_scale == 0

    def loss_scale(self):
        return self._config.loss_scale

    def dynamic_loss_scale_args(self):
        return self._config.dynamic_loss_scale_args

    def gradient_clipping(self):
        return self._config.gradient_clipping

    def zero_optimization(self):
        return self._config.zero_enabled

    def zero_optimization_stage(self):
        return self._config.zero_optimization_stage

    def zero_reduce_bucket_size(self):
        return self._config.zero_reduce_bucket_size

    def zero_overlap_comm(self):
        return self._config.zero_overlap_comm

    def wall_clock_breakdown(self):
        return self._config.wall_clock_breakdown

    def optimizer_name(self):
        return self._config.optimizer_name

    def optimizer_params(self):
        return self._config.optimizer_params

    def gradient_accumulation_steps(self):
        return self._config.gradient_accumulation_steps

    def is_gradient_accumulation_boundary(self):
        return (self.micro_steps + 1) % self.gradient_accumulation_steps() == 0

    # ---- hooks
    def _configure_basic_optimizer(self, model_parameters):
        name = (self.optimizer_name() or 'adamw').lower()
        params = dict(self.optimizer_params())
        params.pop('torch_adam', None)
        cls = {'adam': torch.optim.Adam, 'adamw': torch.optim.AdamW}[name]
        return cls(model_parameters if model_parameters is not None else self.module.parameters(), **params)

    def _configure_optimizer(self, client_optimizer, model_parameters):
        self.basic_optimizer = client_optimizer or self._configure_basic_optimizer(model_parameters)
        self.optimizer = self.basic_optimizer

    def _configure_lr_scheduler(self, client_lr_scheduler):
        if client_lr_scheduler is not None:
            self.lr_scheduler = client_lr_scheduler
            return
        name = self._config.scheduler_name
        if name is None:
            return
        p = self._config.scheduler_params
        target = self.optimizer
        if name == 'WarmupDecayLR':    # one of DeepSpeed's schedulers that msamp's stand-alone engine does not implement
            total, warm, hi = p['total_num_steps'], p.get('warmup_num_steps', 0), p.get('warmup_max_lr', 1e-3)

            class _Sched:
                def __init__(self):
                    self.t = 0
                    self._apply()

                def _apply(self):
                    f = (self.t / max(1, warm)) if self.t < warm else max(0.0, (total - self.t) / max(1, total - warm))
                    for g in target.param_groups:
                        g['lr'] = hi * f

                def step(self):
                    self.t += 1
                    self._apply()

                def get_lr(self):
                    return [g['lr'] for g in target.param_groups]

            self.lr_scheduler = _Sched()
        else:
            raise ValueError(name)

    # ---- training loop
    def forward(self, *inputs, **kwargs):
        return self.module(*inputs, **kwargs)

    def allreduce_gradients(self, bucket_size=None):
        raise RuntimeError('the fake engine has no gradient all-reduce: an engine with FP8 gradients must override this')

    def backward(self, loss):
        ga = self.gradient_accumulation_steps()
        if ga > 1:
            loss = loss / ga
        if hasattr(self.optimizer, 'backward'):
            self.optimizer.backward(loss)
        else:
            loss.backward()
        self.allreduce_gradients()
        return loss

    def _take_model_step(self):
        self.optimizer.step()
        overflow = bool(getattr(self.optimizer, 'overflow', False))
        self.optimizer.zero_grad()
        if overflow:
            self.skipped_steps += 1
        elif self.lr_scheduler is not None:
            self.lr_scheduler.step()
        self.global_steps += 1

    def step(self):
        if self.is_gradient_accumulation_boundary():
            self._take_model_step()
        self.micro_steps += 1
