"""Global-norm gradient clipping over mixed Tensor / ScalingTensor gradients.

(reference: msamp/nn/clip_grad.py:11-88).  A ScalingTensor gradient contributes the norm of its
dequantised values and is clipped by scaling its ``scale_inv`` only – its bytes are not touched.
No host synchronisation happens unless ``error_if_nonfinite`` is set.
"""
import torch

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingTensor


def _grad_norm(g, norm_type):
    if isinstance(g, ScalingTensor):
        if Dtypes.is_fp8_qtype(g.qtype):
            from msamp.ops import reduce as _r
            return _r.fp8_norm(g.value, g.qtype, g.meta.scale_inv, norm_type)
        return torch.linalg.vector_norm(g.value.float(), norm_type) * g.meta.scale_inv.float()
    return torch.linalg.vector_norm(g.detach().float(), norm_type)


def _one_device(grads):
    devs = {(g.value if isinstance(g, ScalingTensor) else g).device for g in grads}
    ok = all((g.value if isinstance(g, ScalingTensor) else g).is_contiguous() for g in grads)
    return len(devs) == 1 and ok and all((g.value if isinstance(g, ScalingTensor) else g).dtype in (
        torch.float32, torch.float16, torch.bfloat16, torch.uint8) for g in grads)


@torch.no_grad()
def clip_grad_norm_(parameters, max_norm, norm_type=2.0, error_if_nonfinite=False):
    """Clip the global gradient norm in place and return the norm before clipping."""
    if isinstance(parameters, (torch.Tensor, ScalingTensor)):
        parameters = [parameters]
    grads = [p.grad for p in parameters if p.grad is not None]
    max_norm, norm_type = float(max_norm), float(norm_type)
    if not grads:
        return torch.tensor(0.0)
    device = grads[0].device
    if norm_type == float('inf'):
        norms = []
        for g in grads:
            if isinstance(g, ScalingTensor):
                norms.append(g.float().abs().max().to(device))
            else:
                norms.append(g.detach().abs().max().float().to(device))
        total = torch.stack(norms).max()
    elif norm_type == 2.0 and _one_device(grads):
        # one launch for the norm of all gradients, one for the clip (msamp.ops.multi_tensor)
        from msamp.ops import multi_tensor as _mt
        stats = _mt.grad_sumsq(grads, tag='clip_grad_norm_')
        total = stats[0].sqrt()
        if error_if_nonfinite and not bool(torch.isfinite(total)):
            raise RuntimeError(
                f'The total norm of order {norm_type} for gradients from `parameters` is non-finite, so it cannot be clipped.'
            )
        _mt.clip_by_sumsq(grads, stats[0:1], max_norm, tag='clip_grad_norm_')
        return total
    else:
        total = torch.linalg.vector_norm(torch.stack([_grad_norm(g, norm_type).to(device) for g in grads]), norm_type)
    if error_if_nonfinite and not bool(torch.isfinite(total)):
        raise RuntimeError(
            f'The total norm of order {norm_type} for gradients from `parameters` is non-finite, so it cannot be clipped.'
        )
    coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    for g in grads:
        if isinstance(g, ScalingTensor):
            g.mul_(coef)
        else:
            g.detach().mul_(coef.to(g.device, g.dtype))
    return total
