"""FsdpReplacer: FP8Linear with e4m3 weights whose bytes are exposed as fp32 ``nn.Parameter``s.

torch's FSDP flattens and shards only real ``torch.Tensor`` parameters of a floating dtype, so every FP8
weight is padded to a multiple of four bytes and viewed as fp32; the information needed to undo that
travels as attributes on the parameter (``_original_shape``, ``_padded``, ``_meta``, ``_scaling_metas``).
``F.linear`` recognises such a parameter by its ``_meta`` and reinterprets the bytes.
(reference: msamp/fsdp/replacer.py:12-37)
"""
import torch

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingTensor
from msamp.nn import LinearReplacer


class FsdpReplacer:
    """Prepares a model for sharding of its FP8 weights."""
    @classmethod
    def replace(cls, model):
        model = LinearReplacer.replace(model, weight_qtype=Dtypes.kfloat8_e4m3)
        for _, sub in model.named_modules():
            for name, param in list(sub.named_parameters(recurse=False)):
                if not isinstance(param, ScalingTensor):
                    continue
                data = param.value.reshape(-1)
                padded = (-data.numel()) % 4
                if padded:
                    data = torch.nn.functional.pad(data, (0, padded))
                new_param = torch.nn.Parameter(data.view(torch.float32), requires_grad=param.requires_grad)
                new_param._original_shape = param.shape
                new_param._padded = padded
                new_param._meta = param.meta
                new_param._scaling_metas = param._scaling_metas
                new_param._grad_meta = param._scaling_metas['wgrad']
                sub._parameters.pop(name, None)
                sub.register_parameter(name, new_param)
                # torch FSDP (use_orig_params) puts a plain view of its flat parameter in place of the parameter
                # while forward and backward run; the module re-attaches these attributes to that view
                stash = sub.__dict__.setdefault('_fp8_param_attrs', {})
                stash[name] = {k: getattr(new_param, k) for k in ('_original_shape', '_padded', '_meta', '_scaling_metas', '_grad_meta')}
        return model
