"""TeReplacer: convert a model built from Transformer Engine modules (reference: msamp/te/replacer.py:13-49).

With Transformer Engine installed, every ``te.Linear`` / ``te.LayerNormLinear`` / ``te.LayerNormMLP`` is replaced
by the msamp module of the same shape (weights copied and cast to scaled fp16 ScalingParameters).
msamp modules that are already in the model only get registered.  Afterwards the FP8 parameters are marked as
DDP-ignored and all scaling metas are registered with ``model_state``.
"""
import torch

from msamp.common.dtype import Dtypes
from msamp.nn.parameter import ScalingParameter
from msamp.nn.state import model_state
from msamp.te.modules import MSAMPLayerNormLinear, MSAMPLayerNormMLP, MSAMPLinear, te_available


class TeReplacer:
    """Replaces weights of Transformer-Engine-style modules by ScalingParameters."""
    module_weight_names = {
        MSAMPLinear: ['weight'],
        MSAMPLayerNormLinear: ['weight', 'query_weight', 'key_weight', 'value_weight'],
        MSAMPLayerNormMLP: ['fc1_weight', 'fc2_weight'],
    }

    @staticmethod
    def _te_classes():
        if not te_available():
            return {}
        import transformer_engine.pytorch as te
        return {te.Linear: MSAMPLinear, te.LayerNormLinear: MSAMPLayerNormLinear, te.LayerNormMLP: MSAMPLayerNormMLP}

    @classmethod
    @torch.no_grad()
    def _convert_te_module(cls, mod, target):
        dev = next(mod.parameters()).device
        if target is MSAMPLinear:
            new = MSAMPLinear(mod.in_features, mod.out_features, bias=getattr(mod, 'bias', None) is not None and mod.bias.numel() > 0, device=dev)
        elif target is MSAMPLayerNormLinear:
            new = MSAMPLayerNormLinear(mod.in_features, mod.out_features, eps=getattr(mod, 'eps', 1e-5),
                                       bias=getattr(mod, 'bias', None) is not None and mod.bias.numel() > 0, device=dev)
        else:
            hidden = mod.layer_norm_weight.numel()
            ffn = mod.fc1_weight.shape[0]
            new = MSAMPLayerNormMLP(hidden, ffn, eps=getattr(mod, 'eps', 1e-5), bias=getattr(mod, 'fc1_bias', None) is not None, device=dev)
        for name, p in mod.named_parameters(recurse=False):
            if not hasattr(new, name):
                continue
            dst = getattr(new, name)
            if isinstance(dst, ScalingParameter):
                dst.copy_(p.data.float().cast(Dtypes.kfloat16))
                dst.requires_grad = p.requires_grad
            elif dst is not None and dst.shape == p.shape:
                dst.data.copy_(p.data)
            p.data = torch.tensor([])    # release the old storage
        return new

    @classmethod
    def _replace(cls, model):
        te_map = cls._te_classes()
        for te_cls, target in te_map.items():
            if type(model) is te_cls:
                return cls._convert_te_module(model, target)
        for name, child in list(model.named_children()):
            setattr(model, name, cls._replace(child))
        return model

    @classmethod
    def replace(cls, model):
        model = cls._replace(model)
        names = [k for k, p in model.named_parameters() if isinstance(p, ScalingParameter)]
        torch.nn.parallel.DistributedDataParallel._set_params_and_buffers_to_ignore_for_model(model, names)
        model_state.register_scaling_metas(model, None)
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        return model
