"""Config object with DeepSpeed's method names (``_initialize_params``, ``_do_error_check``) and attribute names."""


class DeepSpeedConfig:
    def __init__(self, config, mpu=None):
        if not isinstance(config, dict):
            raise ValueError('the fake config takes a dict')
        self._param_dict = config
        self.world_size = mpu.get_data_parallel_world_size() if mpu is not None else 1
        self._initialize_params(config)
        self._configure_train_batch_size()
        self._do_error_check()

    def _initialize_params(self, d):
        self.train_batch_size = d.get('train_batch_size')
        self.train_micro_batch_size_per_gpu = d.get('train_micro_batch_size_per_gpu')
        self.gradient_accumulation_steps = d.get('gradient_accumulation_steps')
        self.gradient_clipping = float(d.get('gradient_clipping', 0.0))
        self.wall_clock_breakdown = bool(d.get('wall_clock_breakdown', False))
        opt = d.get('optimizer') or {}
        self.optimizer_name = opt.get('type')
        self.optimizer_params = dict(opt.get('params') or {})
        sch = d.get('scheduler') or {}
        self.scheduler_name = sch.get('type')
        self.scheduler_params = dict(sch.get('params') or {})
        fp16 = d.get('fp16') or {}
        self.fp16_enabled = bool(fp16.get('enabled', False))
        self.loss_scale = float(fp16.get('loss_scale', 0))
        self.dynamic_loss_scale_args = dict(init_scale=2**int(fp16.get('initial_scale_power', 16)), scale_window=int(fp16.get('loss_scale_window', 1000)),
                                            min_scale=float(fp16.get('min_loss_scale', 1)), delayed_shift=int(fp16.get('hysteresis', 2)))
        zero = d.get('zero_optimization') or {}
        self.zero_optimization_stage = int(zero.get('stage', 0))
        self.zero_enabled = self.zero_optimization_stage > 0
        self.zero_reduce_bucket_size = int(zero.get('reduce_bucket_size', 5e8))
        self.zero_overlap_comm = bool(zero.get('overlap_comm', False))

    def _configure_train_batch_size(self):
        mb = self.train_micro_batch_size_per_gpu or 1
        ga = self.gradient_accumulation_steps or 1
        self.train_micro_batch_size_per_gpu, self.gradient_accumulation_steps = mb, ga
        self.train_batch_size = self.train_batch_size or mb * ga * self.world_size

    def _do_error_check(self):
        assert self.train_batch_size == self.train_micro_batch_size_per_gpu * self.gradient_accumulation_steps * self.world_size
