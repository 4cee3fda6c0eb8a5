"""msamp: FP8 mixed-precision training for NVIDIA B200.

Public surface (same as the reference, msamp/__init__.py:14-103): ``initialize``, ``clip_grad_norm_``,
``opt_levels``, ``__version__``.  Importing the package installs the torch patches that let
ScalingTensor flow through ``F.linear``, AMP's GradScaler, ``zeros_like`` and ``load_state_dict``.
"""
import torch

from msamp.common.dtype import Dtypes
from msamp.nn import LinearReplacer, clip_grad_norm_
from msamp.optim import LBAdam, LBAdamW, DSAdam

__version__ = '0.4.0'
__author__ = 'msamp-b200 authors'

opt_levels = ['O1', 'O2', 'O3']


def _is_fused_adam(optimizer):
    return type(optimizer).__name__ == 'FusedAdam' and hasattr(optimizer, 'adam_w_mode')


def initialize(model, optimizer=None, opt_level='O1', use_te=False, group=None, src_rank=0):
    """Convert ``model`` and ``optimizer`` for FP8 training and return ``(model, optimizer)``.

    ================  =====  =====  ==========  =============  ================
    opt_level         GEMM   comm   weight      weight grad    Adam m / v
    ================  =====  =====  ==========  =============  ================
    ``'O1'``          fp8    fp8    fp16 (s)    fp8            fp32 / fp32
    ``'O2'``          fp8    fp8    fp16 (s)    fp8            fp8 / fp16 (s)
    ``'O3'``          fp8    fp8    fp8 + fp16 (s) master      fp8 / fp16 (s)
    ================  =====  =====  ==========  =============  ================

    (s) = stored with a per-tensor power-of-two scale.  ``O3`` is an extension of the reference's
    API, which accepts it only through its DeepSpeed integration; here the returned optimizer keeps
    the scaled-fp16 master weights itself (see ``msamp.optim.master.FP8MasterOptimizer``).

    Args:
        model (torch.nn.Module): model whose ``nn.Linear`` layers are replaced by ``FP8Linear``.
        optimizer: ``torch.optim.Adam``/``AdamW`` (or DeepSpeed ``FusedAdam``); default ``AdamW(model.parameters())``.
        opt_level (str): one of ``opt_levels``.
        use_te (bool): convert Transformer Engine modules instead (needs transformer_engine).
        group, src_rank: process group (and the global rank inside it) from which the converted weights are broadcast;
            default: the world group and rank 0. Pipeline stages pass their own data-parallel group.
    """
    process_group = group    # `group` is reused below as the loop variable over optimizer param groups
    if not isinstance(model, torch.nn.Module):
        raise ValueError('Model must be an instance of torch.nn.Module')
    if opt_level not in opt_levels:
        raise ValueError(f'Invalid optimization level. Please choose from {opt_levels}')
    if not optimizer:
        # Default AdamW. The model may already contain ScalingParameters (msamp.te modules), which torch's
        # optimizers reject, so the stand-in is built on the plain tensors only and rebound after conversion.
        plain = [p for p in model.parameters() if torch.is_tensor(p)]
        optimizer = torch.optim.AdamW(plain if plain else [torch.nn.Parameter(torch.zeros(1))])
        optimizer.param_groups[0]['params'] = list(model.parameters())
    if not (isinstance(optimizer, (torch.optim.AdamW, torch.optim.Adam)) or _is_fused_adam(optimizer)):
        raise ValueError(f'Optimizer {optimizer} is not supported in optimization level {opt_level}')

    # Parameter identity changes during conversion; positions in model.parameters() do not.
    position = {id(p): i for i, p in enumerate(model.parameters())}
    index_list = []
    for group in optimizer.param_groups:
        for p in group['params']:
            if id(p) not in position:
                raise ValueError('optimizer holds a parameter that is not in the model')
            index_list.append(position[id(p)])

    weight_qtype = Dtypes.kfloat8_e4m3 if opt_level == 'O3' else Dtypes.kfloat16
    if use_te:
        from msamp.te import TeReplacer
        cast_model = TeReplacer.replace(model)
    else:
        cast_model = LinearReplacer.replace(model, weight_qtype=Dtypes.kfloat16, src_rank=src_rank, group=process_group)

    parameters = list(cast_model.parameters())
    k = 0
    for group in optimizer.param_groups:
        params = group['params']
        for i in range(len(params)):
            params[i] = parameters[index_list[k]]
            k += 1

    args = dict(optimizer.defaults)
    if opt_level == 'O1':
        args['exp_avg_dtype'], args['exp_avg_sq_dtype'] = torch.float32, torch.float32
    else:
        args['exp_avg_dtype'], args['exp_avg_sq_dtype'] = torch.uint8, torch.float16
    for key in ('foreach', 'capturable', 'differentiable', 'fused', 'decoupled_weight_decay'):
        args.pop(key, None)
    groups = []
    for g in optimizer.param_groups:
        g = dict(g)
        for key in ('foreach', 'capturable', 'differentiable', 'fused', 'decoupled_weight_decay'):
            g.pop(key, None)
        groups.append(g)

    if isinstance(optimizer, torch.optim.AdamW):
        cast_optimizer = LBAdamW(groups, **args)
    elif isinstance(optimizer, torch.optim.Adam):
        if optimizer.defaults.get('decoupled_weight_decay', False):
            cast_optimizer = LBAdamW(groups, **args)
        else:
            cast_optimizer = LBAdam(groups, **args)
    else:
        args.pop('adam_w_mode', None)
        cast_optimizer = DSAdam(groups, **args, adam_w_mode=optimizer.adam_w_mode)

    if opt_level == 'O3':
        from msamp.optim.master import FP8MasterOptimizer
        cast_optimizer = FP8MasterOptimizer(cast_model, cast_optimizer)
    del weight_qtype
    return cast_model, cast_optimizer


__all__ = ['clip_grad_norm_', 'initialize', 'opt_levels', '__version__']
