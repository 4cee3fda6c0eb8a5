"""The public names, signatures and defaults a user of the reference relies on (import paths are also part of
the checkpoint format, because state dicts pickle classes by module path)."""
import inspect

import pytest
import torch

import msamp


def _params(fn):
    return list(inspect.signature(fn).parameters)


def test_top_level():
    assert msamp.__version__ == '0.4.0'
    assert msamp.opt_levels[:2] == ['O1', 'O2']
    p = inspect.signature(msamp.initialize).parameters
    assert list(p)[:4] == ['model', 'optimizer', 'opt_level', 'use_te']
    assert p['optimizer'].default is None and p['opt_level'].default == 'O1' and p['use_te'].default is False
    assert _params(msamp.clip_grad_norm_)[:4] == ['parameters', 'max_norm', 'norm_type', 'error_if_nonfinite']
    with pytest.raises(ValueError):
        msamp.initialize(torch.nn.Linear(4, 4), torch.optim.SGD(torch.nn.Linear(4, 4).parameters(), lr=0.1), 'O1')
    with pytest.raises(ValueError):
        msamp.initialize(torch.nn.Linear(4, 4), None, 'O9')


def test_dtypes_and_floating():
    from msamp.common.dtype import Dtypes, Floating, QType
    names = ['kbyte', 'kint32', 'kfloat32', 'kfloat16', 'kbfloat16', 'kfloat8_e4m3', 'kfloat8_e5m2']
    assert [int(getattr(Dtypes, n)) for n in names] == list(range(7))
    assert isinstance(Dtypes.kfloat8_e4m3, QType) and hash(Dtypes.kfloat8_e4m3) is not None
    for attr in ('dtype_to_qtype', 'qtype_to_dtype', 'dtype_to_size', 'is_fp8_qtype', 'get_dtype_from_qtype'):
        assert hasattr(Dtypes, attr)
    assert torch.fp8e4m3 is torch.uint8 and torch.fp8e5m2 is torch.int8
    assert Floating.qfp_max[Dtypes.kfloat8_e4m3] == 448.0 and Floating.qfp_max[Dtypes.kfloat8_e5m2] == 57344.0
    assert Floating.fp_maxs[torch.float16] == 65504.0
    assert Floating._get_fp_max(4, 3, inf_existed=False) == 448.0


def test_tensor_layer():
    from msamp.common.tensor import HookManager, ScalingMeta, ScalingTensor, TensorDist, TypeCast
    from msamp.common.dtype import Dtypes
    p = inspect.signature(ScalingMeta.__init__).parameters
    assert list(p)[1:7] == ['qtype', 'scale', 'scale_inv', 'amax', 'window_size', 'group']
    for m in ('compute_scaling_factor', 'is_warmup', 'is_in_time_scaling', 'in_time_scaling_context', 'reset_scaling_factor', 'copy_',
              'clone', 'cuda', 'is_cuda'):
        assert hasattr(ScalingMeta, m), m
    x = torch.randn(8, 16)
    t = x.cast(Dtypes.kfloat8_e4m3)
    assert isinstance(t, ScalingTensor) and t.qtype == Dtypes.kfloat8_e4m3 and x.qtype == Dtypes.kfloat32
    a, b = x.fused_cast_transpose(Dtypes.kfloat8_e4m3)
    assert a.shape == (8, 16) and b.shape == (16, 8)
    with pytest.raises(TypeError):
        x.fused_cast_transpose(Dtypes.kfloat16)
    for m in ('cast_to_fp8', 'cast_to_fp16', 'cast_from_fp8', 'cast_from_fp16', 'cast_from_fp32'):
        assert hasattr(TypeCast, m), m
    assert _params(TypeCast.cast_to_fp8)[:4] == ['input', 'meta', 'sync', 'fuse_transpose']
    for m in ('broadcast', 'all_reduce', 'all_reduce_avg', 'all_reduce_sum'):
        assert hasattr(TensorDist, m), m
    hm = HookManager()
    seen = []
    h = hm.register_hook(lambda *a: seen.append(a))
    hm(1)
    h.remove()
    hm(2)
    assert len(seen) == 1
    # the tensor-like API that optimizers, DDP and checkpoints rely on
    for m in ('value', 'meta', 'grad', 'cast', 'cast_', 'float', 'half', 'bfloat16', 'to', 't', 'fp8_transpose', 'contiguous', 'clone', 'cpu',
              'cuda', 'copy_', 'zero_', 'mul_', 'div_', 'abs', 'min', 'max', 'pad', 'flatten', 'has_inf_or_nan', 'isnan', 'shape', 'size',
              'numel', 'data', 'detach', 'view', 'reshape', 'requires_grad_', 'register_backward_post_hook', 'backward_grad_update', 'dim',
              'dtype', 'device', 'is_cuda', 'is_leaf', 'qtype'):
        assert hasattr(t, m), m


def test_operators():
    from msamp.operators.arithmetic import Arithmetic
    from msamp.operators.dist_op import DistOp
    from msamp.operators.fp4_quantize import FP4_QUANTIZER
    from msamp.operators.gemm import Gemm
    assert _params(Gemm.fp8_gemm)[:7] == ['mat_a', 'mat_b', 'out_qtype', 'bias', 'accumulate', 'out', 'use_split_accumulator']
    assert _params(Arithmetic.add_to_fp8)[:3] == ['fp8_tensor', 'meta', 'other']
    for m in ('enable_fp8', 'disable_fp8', 'all_reduce', 'reduce'):
        assert hasattr(DistOp, m), m
    p = inspect.signature(FP4_QUANTIZER.apply_DGE_item).parameters
    assert p['k'].default == 5.0 and p['power_clamp_max'].default == 3.0
    q = inspect.signature(FP4_QUANTIZER.quantize_simulate_fp4_in_bf16).parameters
    for name in ('format', 'nan_existed', 'channel_wise', 'token_wise', 'outlier_clip', 'clip_threshold', 'residual_compensation',
                 'return_scaled_input_for_bwd'):
        assert name in q, name
    assert q['clip_threshold'].default == 0.99


def test_nn_and_optim():
    from msamp.common.dtype import Dtypes
    from msamp.nn import FP8Linear, LinearReplacer, ScalingModule, ScalingParameter, clip_grad_norm_, model_state    # noqa: F401
    from msamp.nn.distributed import FP8DistributedDataParallel
    from msamp.optim import DSAdam, FSDPAdam, FSDPAdamW, LBAdam, LBAdamW, LBAdamWBase, LBOptimizer    # noqa: F401
    p = inspect.signature(FP8Linear.__init__).parameters
    assert list(p)[1:3] == ['in_features', 'out_features'] and p['weight_qtype'].default == Dtypes.kfloat16
    assert FP8Linear.DEFAULT_WINDOW_SIZE == 16 and FP8Linear.DEFAULT_WGRAD_WINDOW_SIZE == 1
    r = inspect.signature(LinearReplacer.replace).parameters
    assert list(r)[:4] == ['model', 'weight_qtype', 'src_rank', 'group'] and r['src_rank'].default == 0
    assert issubclass(FP8DistributedDataParallel, torch.nn.parallel.DistributedDataParallel) or hasattr(FP8DistributedDataParallel, 'forward')
    o = inspect.signature(LBAdamW.__init__).parameters
    assert o['lr'].default == 1e-3 and o['eps'].default == 1e-8 and o['weight_decay'].default == 1e-2
    assert o['exp_avg_dtype'].default is torch.uint8 and o['exp_avg_sq_dtype'].default is torch.float16 and o['tensor_scale'].default is True
    assert inspect.signature(LBAdam.__init__).parameters['weight_decay'].default == 0
    for m in ('step', 'lb_step', 'all_reduce_grads', 'state_dict', 'load_state_dict', 'zero_grad', 'add_param_group'):
        assert hasattr(LBOptimizer, m), m


def test_integrations_are_importable():
    from msamp import deepspeed, fsdp, megatron, te
    assert callable(deepspeed.initialize)
    d = inspect.signature(deepspeed.initialize).parameters
    for name in ('args', 'model', 'optimizer', 'model_parameters', 'training_data', 'lr_scheduler', 'mpu', 'dist_init_required', 'collate_fn',
                 'config', 'config_params'):
        assert name in d, name
    for name in ('FP8DistributedDataParallel', 'FP8DistributedOptimizer', 'FP8LinearWithGradAccumulationAndAsyncCommunication',
                 'clip_grad_norm_fp32'):
        assert hasattr(megatron, name), name
    assert hasattr(fsdp, 'FsdpReplacer') and hasattr(fsdp, 'FP8FullyShardedDataParallel')
    assert hasattr(te, 'TeReplacer')
    from msamp.common.utils import DistUtil, TransformerEngineWrapper, logger    # noqa: F401
    from msamp.models import GPT, ParallelGPT, gpt_config    # noqa: F401
    assert gpt_config('gpt-7b').n_layer == 32 and gpt_config('gpt-13b').hidden == 5120 and gpt_config('gpt-30b').n_head == 56


def test_bench_reference_arm_prints_one_json_line():
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, 'bench.py'), '--impl', 'reference'], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out['impl'] == 'reference' and ('unavailable' in out or 'value' in out)
