"""FP8DeepSpeedZeroOptimizer: ZeRO stage 1/2 for models with FP8 weights.

What the reference's optimizer does (msamp/deepspeed/runtime/zero/fp8_stage_1_and_2.py:26-1023) – whole-tensor greedy
ownership, fp16 masters and low-bit moments only on the owner, a flat padded e4m3 weight buffer on every
rank, FP8 gradient reduction to the owner, FP8-aware overflow handling, ``single_partition_of_fp8_groups`` in
the checkpoint – is provided by ``msamp.parallel.zero.ZeroShardedOptimizer``; this class adds the loss-scaling /
overflow / clipping policy and DeepSpeed's method names.  Stages 1 and 2 differ only in when gradients
could be released; with FP8 gradients stored in one flat buffer both behave identically here.
"""
from msamp.deepspeed.runtime.fp8.fused_optimizer import FP8Optimizer
from msamp.deepspeed.runtime.zero.utils import is_zero_supported_optimizer
from msamp.utils.timer import PhaseTimers

OPTIMIZER_ALLGATHER, OPTIMIZER_GRADIENTS, OPTIMIZER_STEP = 'optimizer_allgather', 'optimizer_gradients', 'optimizer_step'


class FP8DeepSpeedZeroOptimizer(FP8Optimizer):
    """ZeRO-1/2 with FP8 weights, FP8 gradients and sharded low-bit optimizer states."""
    def __init__(self, model, init_optimizer, static_loss_scale=1.0, dynamic_loss_scale=False, dynamic_loss_args=None, clip_grad=0.0,
                 dp_process_group=None, partition_grads=True, mpu=None, timers=None, reduce_bucket_size=500000000, overlap_comm=False):
        if not is_zero_supported_optimizer(init_optimizer):
            raise AssertionError(f'{type(init_optimizer).__name__} is not supported by FP8 ZeRO; use LBAdam/LBAdamW/DSAdam')
        super().__init__(
            model, init_optimizer, static_loss_scale=static_loss_scale, dynamic_loss_scale=dynamic_loss_scale,
            dynamic_loss_args=dynamic_loss_args, clip_grad=clip_grad, fp8_master=True, zero_stage=2 if partition_grads else 1,
            group=dp_process_group, mpu=mpu, timers=timers or PhaseTimers(enabled=False)
        )
        self.partition_gradients = partition_grads
        self.reduce_bucket_size = reduce_bucket_size
        self.overlap_comm = overlap_comm
        self.dp_process_group = dp_process_group

    @property
    def partition_count(self):
        return self.zero.world

    # DeepSpeed's engine calls these between backward and step; here the (fused) reduction of all gradients happens
    # inside step(), so they have nothing left to do.
    def overlapping_partition_gradients_reduce_epilogue(self):
        return None

    def reduce_gradients(self, pipeline_parallel=False):
        return None

    def has_overflow(self, partition_gradients=True):
        return self.overflow_checker.check(self._all_params())

    def state_dict(self):
        sd = super().state_dict()
        # the reference's key and nesting: a list of param groups, each a list of detached master ScalingTensors
        # (msamp/deepspeed/runtime/zero/fp8_stage_1_and_2.py:937-960)
        sd['single_partition_of_fp8_groups'] = sd.get('fp8_master_groups') or []
        sd['partition_count'] = self.partition_count
        sd['zero_stage'] = 2 if self.partition_gradients else 1
        return sd

    def load_state_dict(self, sd, load_optimizer_states=True, load_from_fp32_weights=False):
        if sd.get('partition_count', self.partition_count) != self.partition_count:
            raise ValueError('changing the data-parallel degree of an FP8 ZeRO checkpoint is not supported')
        sd = dict(sd)
        if 'single_partition_of_fp8_groups' in sd:
            saved = sd['single_partition_of_fp8_groups']
            nested = bool(saved) and isinstance(saved[0], (list, tuple))
            sd['fp8_master_groups'] = saved if (nested or not saved) else [saved]    # a flat list is the layout of older files
        super().load_state_dict(sd, load_optimizer_states=load_optimizer_states)
