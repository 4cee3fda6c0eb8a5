"""Global-norm clipping across model-parallel ranks (reference: msamp/megatron/optimizer/clip_grads.py:12-109).

The norm combines high-precision gradients and FP8 ScalingTensor gradients (their dequantised values),
is SUM/MAX-reduced over the model-parallel group, and the clip coefficient multiplies plain tensors
directly and ScalingTensors through their ``scale_inv``.  The only host synchronisation is the final
``.item()`` that Megatron's callers expect.
"""
import torch
import torch.distributed as dist

from msamp.common.tensor import ScalingTensor
from msamp.nn.clip_grad import _grad_norm, _one_device


def clip_grad_norm_fp32(parameters, grads_for_norm, max_norm, norm_type=2, model_parallel_group=None):
    """Clip gradients of ``parameters`` in place using the norm of ``grads_for_norm``; returns the total norm (float).

    Args:
        parameters: tensors / ScalingTensors (or one of them) whose ``.grad`` (or ``main_grad``) gets scaled.
        grads_for_norm: the gradients that count for the norm on this rank (duplicates across TP ranks excluded by the caller).
        max_norm: clipping threshold.
        norm_type: 2 (default), any p > 0, or ``inf``.
        model_parallel_group: group over which the norm is reduced.
    """
    if isinstance(parameters, (torch.Tensor, ScalingTensor)):
        parameters = [parameters]
    if isinstance(grads_for_norm, (torch.Tensor, ScalingTensor)):
        grads_for_norm = [grads_for_norm]
    grads = []
    for p in parameters:
        g = getattr(p, 'main_grad', None) if getattr(p, 'grad', None) is None else p.grad
        if g is not None:
            grads.append(g)
    max_norm, norm_type = float(max_norm), float(norm_type)
    device = None
    for g in list(grads_for_norm) + grads:
        device = g.device
        break
    if device is None:
        return 0.0
    if norm_type == float('inf'):
        vals = [(g.float().abs().max() if isinstance(g, ScalingTensor) else g.detach().abs().max().float()) for g in grads_for_norm]
        total = torch.stack(vals).max() if vals else torch.zeros((), device=device)
        if model_parallel_group is not None and dist.is_initialized():
            dist.all_reduce(total, op=dist.ReduceOp.MAX, group=model_parallel_group)
    elif norm_type == 2.0 and _one_device(list(grads_for_norm) + grads):
        # one launch for the squared norm of every gradient, one for the clip (replaces apex's multi_tensor_l2norm /
        # multi_tensor_scale of the reference, clip_grads.py:79-107)
        from msamp.ops import multi_tensor as _mt
        stats = _mt.grad_sumsq(list(grads_for_norm), out=torch.zeros(2, dtype=torch.float32, device=device), tag='megatron_norm')
        if model_parallel_group is not None and dist.is_initialized():
            dist.all_reduce(stats, op=dist.ReduceOp.SUM, group=model_parallel_group)
        _mt.clip_by_sumsq(grads, stats[0:1], max_norm, eps=1.0e-6, tag='megatron_clip')
        return stats[0].sqrt().item()
    else:
        acc = torch.zeros((), dtype=torch.float32, device=device)
        for g in grads_for_norm:
            acc += _grad_norm(g, norm_type)**norm_type
        if model_parallel_group is not None and dist.is_initialized():
            dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=model_parallel_group)
        total = acc**(1.0 / norm_type)
    coef = max_norm / (total + 1.0e-6)
    clipped = torch.clamp(coef, max=1.0)
    for g in grads:
        if isinstance(g, ScalingTensor):
            g.mul_(clipped)
        else:
            g.detach().mul_(clipped.to(g.dtype))
    return total.item()
