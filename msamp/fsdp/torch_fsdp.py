"""FP8 weights under torch's own FullyShardedDataParallel, through its public hooks.

The reference makes torch FSDP carry FP8 bytes by replacing the private ``FlatParamHandle`` class and the
private ``_post_backward_hook`` (msamp/fsdp/flat_param.py:10-65, msamp/fsdp/_runtime_utils.py:10-26,
msamp/fsdp/fully_sharded_data_parallel.py:14-63).  Current torch needs neither patch:

* ``use_orig_params=True`` keeps the original ``nn.Parameter`` objects, so the attributes that
  ``FsdpReplacer`` attaches (``_meta``, ``_grad_meta``, ``_original_shape``, ``_padded``,
  ``_scaling_metas``) survive flattening and are seen by ``F.linear`` and by ``FSDPAdamW``;
* ``register_comm_hook`` is the public place for a custom gradient reduction.

The hook below treats the flat gradient segment by segment: the bytes of an FP8 weight gradient (all
ranks quantised it with one scale, because the amax was MAX-reduced first) are summed as FP8 numbers
and the mean is taken by dividing the gradient's ``scale_inv``; every other segment is averaged in
its own dtype.  Each rank then keeps its shard.  ``msamp.fsdp.FP8FullyShardedDataParallel`` is the
B200-first alternative that shards by rows and fuses the parameter gather into the GEMM.
"""
import torch
import torch.distributed as dist

from msamp.common.dtype import Dtypes
from msamp.fsdp.replacer import FsdpReplacer
from msamp.operators.dist_op import DistOp


def _segments(flat_param):
    """``(start, end, param or None)`` for every piece of the unsharded flat parameter (None = alignment padding)."""
    numels = getattr(flat_param, '_numels_with_padding', None)
    mask = getattr(flat_param, '_is_padding_mask', None)
    params = list(flat_param._params)
    if numels is None or mask is None:
        numels, mask = flat_param._numels, [False] * len(flat_param._numels)
    out, start, k = [], 0, 0
    for n, is_pad in zip(numels, mask):
        if is_pad:
            out.append((start, start + n, None))
        else:
            out.append((start, start + n, params[k]))
            k += 1
        start += n
    return out


def make_fp8_comm_hook(fsdp_module):
    """Gradient hook of one FSDP instance: FP8 segments are reduced as FP8, the rest as usual, then sharded."""
    def hook(state, grad, output=None):
        group = fsdp_module.process_group
        world = dist.get_world_size(group)
        rank = dist.get_rank(group)
        handle = getattr(fsdp_module, '_handle', None)
        flat = handle.flat_param if handle is not None else None
        segs = _segments(flat) if flat is not None else []
        if not any(p is not None and getattr(p, '_meta', None) is not None for _, _, p in segs):
            grad.div_(world)
            if output is None:    # NO_SHARD: plain all-reduce
                dist.all_reduce(grad, group=group)
            else:
                dist.all_reduce(grad, group=group)
                n = output.numel()
                output.copy_(grad[rank * n:(rank + 1) * n])
            return
        for start, end, p in segs:
            if p is None or end <= start:
                continue
            piece = grad[start:end]
            gmeta = getattr(p, '_grad_meta', None)
            if getattr(p, '_meta', None) is not None and gmeta is not None:
                raw = piece.view(Dtypes.get_dtype_from_qtype(gmeta.qtype))
                DistOp.all_reduce(raw, gmeta.qtype, dist.ReduceOp.SUM, group)
            else:
                dist.all_reduce(piece, group=group)
                piece.div_(world)
        # the mean of the FP8 sums goes into the scale (once per gradient tensor)
        seen = set()
        for _, _, p in segs:
            gmeta = getattr(p, '_grad_meta', None) if p is not None else None
            if gmeta is not None and getattr(p, '_meta', None) is not None and id(gmeta) not in seen:
                seen.add(id(gmeta))
                gmeta.scale_inv.div_(world)
        if output is not None:
            n = output.numel()
            output.copy_(grad[rank * n:(rank + 1) * n])

    return hook


def wrap_with_torch_fsdp(model, **fsdp_kwargs):
    """``FsdpReplacer.replace`` + ``torch.distributed.fsdp.FullyShardedDataParallel`` + the FP8 gradient hook.

    Returns the FSDP module; build the optimizer with ``msamp.optim.FSDPAdamW(fsdp.parameters(), ...)`` afterwards.
    Gradient accumulation across several backward passes is not supported for FP8 parameters (neither is it in the
    reference: the second gradient would have to be added in FP8 with a fresh scale).
    """
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
    model = FsdpReplacer.replace(model)
    fsdp_kwargs['use_orig_params'] = True
    fsdp = FSDP(model, **fsdp_kwargs)
    for sub in FSDP.fsdp_modules(fsdp):
        sub.register_comm_hook(None, make_fp8_comm_hook(sub))
    return fsdp


__all__ = ['wrap_with_torch_fsdp', 'make_fp8_comm_hook']
