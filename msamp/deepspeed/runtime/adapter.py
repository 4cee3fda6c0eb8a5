"""Adapter for an installed DeepSpeed: ``DeepSpeedEngine`` / ``DeepSpeedConfig`` subclasses wired to msamp's FP8 optimizers.

When ``deepspeed`` imports, ``msamp.deepspeed.initialize`` returns an engine built by the classes made here, so that
everything DeepSpeed's own engine provides (its optimizer and scheduler zoo, monitors, activation-checkpointing
config, data loader, checkpoint layout, MoE process groups) keeps working, and only the pieces that touch FP8 tensors
are replaced - the same cut as the reference's ``MSAMPDeepSpeedEngine(DeepSpeedEngine)``
(msamp/deepspeed/runtime/engine.py:61-486) and ``MSAMPDeepSpeedConfig(DeepSpeedConfig)`` (.../config.py:58-86):

* ``_configure_optimizer``: the basic optimizer DeepSpeed would have built is passed through ``msamp.initialize``
  (model conversion + LBAdam/LBAdamW), then wrapped by ``FP8DeepSpeedZeroOptimizer`` (ZeRO 1/2) or ``FP8Optimizer``;
* ``allreduce_gradients``: a no-op, because both wrappers exchange gradients inside ``step()`` (fused FP8 reduction);
* the config additionally parses the ``"msamp"`` section and applies the reference's O3-needs-ZeRO check.

Without DeepSpeed, ``msamp.deepspeed`` falls back to its stand-alone engine (``runtime/engine.py``).
The classes are created lazily because their base classes only exist when DeepSpeed does.
"""
import importlib
import importlib.util

import torch.distributed as dist

import msamp
from msamp.deepspeed.runtime.config import get_msamp_enabled, get_msamp_optlevel, get_msamp_use_te


def deepspeed_available():
    """True if a ``deepspeed`` package with ``runtime.engine.DeepSpeedEngine`` can be imported."""
    try:
        if importlib.util.find_spec('deepspeed') is None:
            return False
        engine = importlib.import_module('deepspeed.runtime.engine')
        return hasattr(engine, 'DeepSpeedEngine')
    except Exception:
        return False


def make_config_class():
    """``DeepSpeedConfig`` subclass that also understands ``"msamp": {"enabled", "opt_level", "use_te"}``."""
    from deepspeed.runtime.config import DeepSpeedConfig

    class MSAMPDeepSpeedConfigAdapter(DeepSpeedConfig):
        def _initialize_params(self, param_dict):
            super()._initialize_params(param_dict)
            self.msamp_enabled = get_msamp_enabled(param_dict)
            self.msamp_optlevel = get_msamp_optlevel(param_dict)
            self.msamp_use_te = get_msamp_use_te(param_dict)

        def _do_error_check(self):
            super()._do_error_check()
            if not self.msamp_enabled:
                return
            assert self.msamp_optlevel in ['O1', 'O2', 'O3'], \
                f'Invalid MS-AMP opt_level: {self.msamp_optlevel}, only O1, O2, O3 are supported.'
            if self.msamp_optlevel == 'O3':
                stage = getattr(self, 'zero_optimization_stage', 0)
                assert getattr(self, 'zero_enabled', stage > 0) and stage in (1, 2), \
                    'MS-AMP O3 requires ZeRO with optimizer_states or gradients partitioning.'

    return MSAMPDeepSpeedConfigAdapter


def make_engine_class():
    """``DeepSpeedEngine`` subclass whose optimizer is one of msamp's FP8 wrappers."""
    from deepspeed.runtime.engine import DeepSpeedEngine
    from msamp.deepspeed.runtime.fp8.fused_optimizer import FP8Optimizer
    from msamp.deepspeed.runtime.zero.fp8_stage_1_and_2 import FP8DeepSpeedZeroOptimizer

    class MSAMPDeepSpeedEngineAdapter(DeepSpeedEngine):
        def msamp_enabled(self):
            return bool(getattr(self._config, 'msamp_enabled', False))

        def msamp_optlevel(self):
            return getattr(self._config, 'msamp_optlevel', None)

        def msamp_use_te(self):
            return bool(getattr(self._config, 'msamp_use_te', False))

        def _dp_group(self):
            mpu = getattr(self, 'mpu', None)
            if mpu is not None and hasattr(mpu, 'get_data_parallel_group'):
                return mpu.get_data_parallel_group()
            getter = getattr(self, 'seq_data_parallel_group', None)    # DeepSpeed >= 0.10 keeps it on the engine
            return getter if (getter is not None and not callable(getter)) else None

        def _configure_optimizer(self, client_optimizer, model_parameters):
            if not self.msamp_enabled():
                return super()._configure_optimizer(client_optimizer, model_parameters)
            if client_optimizer is not None and not callable(client_optimizer):
                basic = client_optimizer
            elif callable(client_optimizer):
                basic = client_optimizer(model_parameters)
            else:
                from msamp.deepspeed.runtime.engine import build_over_all_parameters
                basic = build_over_all_parameters(self._configure_basic_optimizer, model_parameters, self.module)    # DeepSpeed's own builder
            level = self.msamp_optlevel()
            init_level = 'O2' if level == 'O3' else level    # the ZeRO wrapper below provides O3's FP8 weights + fp16 masters
            group = self._dp_group()
            src = dist.get_global_rank(group, 0) if (group is not None and dist.is_initialized()) else 0
            self.module, lb_opt = msamp.initialize(self.module, basic, init_level, use_te=self.msamp_use_te(), group=group, src_rank=src)
            self.basic_optimizer = lb_opt
            dynamic = bool(self.fp16_enabled() and self.dynamic_loss_scale())
            static = self.loss_scale() if (self.fp16_enabled() and not dynamic) else 1.0
            dyn_args = self.dynamic_loss_scale_args() if dynamic else None
            if isinstance(dyn_args, dict):    # DeepSpeed's names -> the FP8 loss scaler's
                dyn_args = dict(init_scale=dyn_args.get('init_scale', 2**16), scale_window=dyn_args.get('scale_window', 1000),
                                min_scale=dyn_args.get('min_scale', 1), delayed_shift=dyn_args.get('delayed_shift', 2))
            clip = self.gradient_clipping()
            timers = self.timers if getattr(self, 'wall_clock_breakdown', lambda: False)() else None
            if self.zero_optimization():
                stage = self.zero_optimization_stage()
                if stage > 2:
                    raise NotImplementedError('ZeRO stage 3 with FP8 is provided by msamp.fsdp.FP8FullyShardedDataParallel')
                self.optimizer = FP8DeepSpeedZeroOptimizer(
                    self.module, lb_opt, static_loss_scale=static, dynamic_loss_scale=dynamic, dynamic_loss_args=dyn_args, clip_grad=clip,
                    dp_process_group=group, partition_grads=stage == 2, mpu=getattr(self, 'mpu', None), timers=timers,
                    reduce_bucket_size=self.zero_reduce_bucket_size(), overlap_comm=self.zero_overlap_comm()
                )
            else:
                self.optimizer = FP8Optimizer(
                    self.module, lb_opt, static_loss_scale=static, dynamic_loss_scale=dynamic, dynamic_loss_args=dyn_args, clip_grad=clip,
                    fp8_master=(level == 'O3'), zero_stage=0, group=group, mpu=getattr(self, 'mpu', None), timers=timers
                )
                world = dist.get_world_size(group) if dist.is_initialized() else 1
                if self.optimizer.zero is None and world > 1:
                    from msamp.parallel.zero import ZeroShardedOptimizer
                    self.optimizer.zero = ZeroShardedOptimizer(self.module, lb_opt, stage=0, group=group)
            # the rest of what DeepSpeed's _configure_optimizer sets up, when the installed version has it
            for name, maker in (('compression_scheduler', '_configure_compression_scheduler'), ('quantizer', '_configure_quantization')):
                if hasattr(self, maker):
                    setattr(self, name, getattr(self, maker)())

        def allreduce_gradients(self, bucket_size=None):
            if not self.msamp_enabled():
                return super().allreduce_gradients(bucket_size) if bucket_size is not None else super().allreduce_gradients()
            # FP8Optimizer / FP8DeepSpeedZeroOptimizer reduce (FP8 and high-precision) gradients inside step()

    return MSAMPDeepSpeedEngineAdapter
