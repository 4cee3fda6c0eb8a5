"""ScalingTensor-aware versions of the cast helpers Transformer Engine modules call.

The reference monkey-patches ``transformer_engine.pytorch.cpp_extensions`` so that TE's own modules accept
ScalingTensor weights (msamp/te/extension.py:15-155).  The same four helpers are provided here as plain
functions; ``TeExtensionOverrider.override()`` installs them into Transformer Engine when it is present.
"""
import torch

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingTensor
from msamp.ops import cast as _k


def _qtype_of(fp8_dtype):
    name = getattr(fp8_dtype, 'name', str(fp8_dtype))
    return Dtypes.kfloat8_e5m2 if 'E5M2' in name.upper() else Dtypes.kfloat8_e4m3


def fused_cast_transpose(inp, fp8_meta_tensor, fp8_tensor, otype, cast_out=None, transpose_out=None):
    """Cast + transpose; a ScalingTensor input is re-quantised from its stored amax instead of being scanned again."""
    qtype = _qtype_of(otype)
    if isinstance(inp, ScalingTensor):
        q = inp.cast(qtype)
        out, out_t = q.value, _k.transpose_fp8(q.value.reshape(-1, q.value.shape[-1]))
        fp8_meta_tensor.scale_inv[fp8_tensor] = q.meta.scale_inv
    else:
        scale = fp8_meta_tensor.scale[fp8_tensor]
        amax = fp8_meta_tensor.amax_history[0][fp8_tensor]
        sinv = fp8_meta_tensor.scale_inv[fp8_tensor]
        out, out_t = _k.cast_transpose_fp8(inp.reshape(-1, inp.shape[-1]), qtype, scale, amax_out=amax, scale_inv_out=sinv)
    if cast_out is not None:
        cast_out.copy_(out.view_as(cast_out))
        transpose_out.copy_(out_t.view_as(transpose_out))
        return None
    return out, out_t


def cast_to_fp8(inp, fp8_meta_tensor, fp8_tensor, otype, out=None):
    qtype = _qtype_of(otype)
    if isinstance(inp, ScalingTensor):
        q = inp.cast(qtype)
        fp8_meta_tensor.scale_inv[fp8_tensor] = q.meta.scale_inv
        res = q.value
    else:
        res = _k.cast_to_fp8(inp, qtype, fp8_meta_tensor.scale[fp8_tensor], amax_out=fp8_meta_tensor.amax_history[0][fp8_tensor],
                             scale_inv_out=fp8_meta_tensor.scale_inv[fp8_tensor])
    if out is not None:
        out.copy_(res.view_as(out))
        return None
    return res


def cast_if_needed(tensor, dtype):
    """TE's helper leaves ScalingTensors alone (they are consumed by the FP8 casts above)."""
    if isinstance(tensor, ScalingTensor):
        return tensor
    return tensor if tensor is None or tensor.dtype == dtype else tensor.to(dtype)


class TeExtensionOverrider:
    """Installs the helpers above into Transformer Engine, if it is importable."""
    installed = False

    @classmethod
    def override(cls):
        try:
            import transformer_engine.pytorch.cpp_extensions as ext    # type: ignore
            import transformer_engine.pytorch.utils as te_utils    # type: ignore
        except Exception:
            return False
        ext.fp8_cast_transpose_fused = fused_cast_transpose
        ext.cast_to_fp8 = cast_to_fp8
        te_utils.cast_if_needed = cast_if_needed
        cls.installed = True
        return True


TeExtensionOverrider.override()

__all__ = ['fused_cast_transpose', 'cast_to_fp8', 'cast_if_needed', 'TeExtensionOverrider', 'torch']
