"""Configuration with the ``msamp`` section (reference: msamp/deepspeed/runtime/config.py:10-86).

Only the keys the engines use are interpreted; unknown keys are kept in ``raw`` untouched.
"""
from msamp.common.utils.dist import DistUtil

MSAMP = 'msamp'
MSAMP_ENABLED = 'enabled'
MSAMP_ENABLED_DEFAULT = False
MSAMP_OPTLEVEL = 'opt_level'
MSAMP_OPTLEVEL_DEFAULT = 'O1'
MSAMP_USE_TE = 'use_te'
MSAMP_USE_TE_DEFAULT = False
FP8 = 'fp8'


def get_msamp_enabled(param_dict):
    return bool(param_dict.get(MSAMP, {}).get(MSAMP_ENABLED, MSAMP_ENABLED_DEFAULT)) if MSAMP in param_dict else False


def get_msamp_optlevel(param_dict):
    return param_dict[MSAMP].get(MSAMP_OPTLEVEL, MSAMP_OPTLEVEL_DEFAULT) if MSAMP in param_dict else None


def get_msamp_use_te(param_dict):
    return param_dict[MSAMP].get(MSAMP_USE_TE, MSAMP_USE_TE_DEFAULT) if MSAMP in param_dict else None


class MSAMPDeepSpeedConfig:
    """Parsed training configuration."""
    def __init__(self, config, mpu=None):
        if not isinstance(config, dict):
            raise ValueError('config must be a dict (or a path, resolved by initialize)')
        self.raw = config
        self._initialize_params(config)
        world = mpu.get_data_parallel_world_size() if mpu is not None and hasattr(mpu, 'get_data_parallel_world_size') else DistUtil.get_world_size()
        self.world_size = world
        self._configure_batch(world)
        self._do_error_check()

    def _initialize_params(self, d):
        self.train_batch_size = d.get('train_batch_size')
        self.train_micro_batch_size_per_gpu = d.get('train_micro_batch_size_per_gpu')
        self.gradient_accumulation_steps = d.get('gradient_accumulation_steps')
        self.steps_per_print = d.get('steps_per_print', 10)
        self.gradient_clipping = float(d.get('gradient_clipping', 0.0))
        self.wall_clock_breakdown = bool(d.get('wall_clock_breakdown', False))
        self.optimizer_name = (d.get('optimizer') or {}).get('type')
        self.optimizer_params = dict((d.get('optimizer') or {}).get('params') or {})
        self.scheduler_name = (d.get('scheduler') or {}).get('type')
        self.scheduler_params = dict((d.get('scheduler') or {}).get('params') or {})
        fp16 = d.get('fp16') or {}
        self.fp16_enabled = bool(fp16.get('enabled', False))
        self.loss_scale = float(fp16.get('loss_scale', 0))
        self.initial_scale_power = int(fp16.get('initial_scale_power', 16))
        self.loss_scale_window = int(fp16.get('loss_scale_window', 1000))
        self.hysteresis = int(fp16.get('hysteresis', 2))
        self.min_loss_scale = float(fp16.get('min_loss_scale', 1))
        self.bf16_enabled = bool((d.get('bf16') or d.get('bfloat16') or {}).get('enabled', False))
        zero = d.get('zero_optimization') or {}
        self.zero_optimization_stage = int(zero.get('stage', 0)) if isinstance(zero, dict) else int(bool(zero))
        self.zero_enabled = self.zero_optimization_stage > 0
        self.zero_reduce_bucket_size = int(zero.get('reduce_bucket_size', 5e8)) if isinstance(zero, dict) else int(5e8)
        self.zero_overlap_comm = bool(zero.get('overlap_comm', False)) if isinstance(zero, dict) else False
        self.msamp_enabled = get_msamp_enabled(d)
        self.msamp_optlevel = get_msamp_optlevel(d)
        self.msamp_use_te = get_msamp_use_te(d)

    def _configure_batch(self, world):
        tb, mb, ga = self.train_batch_size, self.train_micro_batch_size_per_gpu, self.gradient_accumulation_steps
        if tb is not None and mb is not None and ga is None:
            ga = tb // (mb * world)
        elif tb is not None and ga is not None and mb is None:
            mb = tb // (ga * world)
        elif mb is not None and tb is None:
            ga = ga or 1
            tb = mb * ga * world
        elif tb is not None and mb is None and ga is None:
            ga = 1
            mb = tb // world
        elif tb is None and mb is None:
            raise AssertionError('Either train_batch_size or train_micro_batch_size_per_gpu needs to be provided')
        self.train_batch_size, self.train_micro_batch_size_per_gpu, self.gradient_accumulation_steps = tb, mb, ga

    def _do_error_check(self):
        tb, mb, ga = self.train_batch_size, self.train_micro_batch_size_per_gpu, self.gradient_accumulation_steps
        assert mb > 0 and ga > 0 and tb > 0, 'batch sizes must be positive'
        assert tb == mb * ga * self.world_size, (
            f'Check batch related parameters. train_batch_size is not equal to micro_batch_per_gpu * gradient_acc_step * world_size '
            f'{tb} != {mb} * {ga} * {self.world_size}'
        )
        assert not (self.fp16_enabled and self.bf16_enabled), 'fp16 and bf16 modes cannot be simultaneously enabled'
        if not self.msamp_enabled:
            return
        assert self.msamp_optlevel in ['O1', 'O2', 'O3'], f'Invalid MS-AMP opt_level: {self.msamp_optlevel}, only O1, O2, O3 are supported.'
        if self.msamp_optlevel == 'O3':
            assert self.zero_enabled and self.zero_optimization_stage in (1, 2), \
                'MS-AMP O3 requires ZeRO with optimizer_states or gradients partitioning.'
