"""FP8Linear and the pass that swaps it in for ``torch.nn.Linear``.

(reference: msamp/nn/linear.py:14-197)
"""
import torch
import torch.nn.functional as F

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingMeta, ScalingTensor, TensorDist
from msamp.common.utils.device import default_device
from msamp.nn.module import ScalingModule
from msamp.nn.parameter import ScalingParameter
from msamp.nn.state import model_state


class FP8Linear(ScalingModule):
    """``y = x Wᵀ + b`` with FP8 GEMMs.

    The weight is a ScalingParameter (scaled fp16 by default, e4m3 at O3); three metas drive the
    quantisation of the GEMM operands: ``input`` (e4m3, window 16), ``wgrad`` (e4m3, window 1) and
    ``ograd`` (e5m2, window 16).
    """
    DEFAULT_WINDOW_SIZE = 16
    DEFAULT_WGRAD_WINDOW_SIZE = 1

    def __init__(self, in_features, out_features, use_bias=True, weight_qtype=Dtypes.kfloat16, bias_type=torch.float32, device=None):
        super().__init__()
        device = torch.device(device) if device is not None else torch.device('cpu')
        self.in_features = in_features
        self.out_features = out_features
        self.weight_qtye = weight_qtype    # (sic) attribute name kept for compatibility
        weight_dtype = Dtypes.get_dtype_from_qtype(weight_qtype)
        value = torch.empty((out_features, in_features), dtype=weight_dtype, device=device)
        self.weight = ScalingParameter(ScalingTensor(value, ScalingMeta(weight_qtype, window_size=1, device=device)))
        if use_bias:
            self.bias = torch.nn.Parameter(torch.empty(out_features, dtype=bias_type, device=device))
        else:
            self.register_parameter('bias', None)
        self.scaling_metas = dict(
            input=ScalingMeta(Dtypes.kfloat8_e4m3, window_size=FP8Linear.DEFAULT_WINDOW_SIZE, device=device),
            wgrad=ScalingMeta(Dtypes.kfloat8_e4m3, window_size=FP8Linear.DEFAULT_WGRAD_WINDOW_SIZE, device=device),
            ograd=ScalingMeta(Dtypes.kfloat8_e5m2, window_size=FP8Linear.DEFAULT_WINDOW_SIZE, device=device),
        )
        self.weight._scaling_metas = self.scaling_metas

    def _apply(self, fn, recurse=True):
        super()._apply(fn, recurse)
        # keep the metas on the weight's device (they are not parameters or buffers)
        dev = self.weight.device
        for m in self.scaling_metas.values():
            if m.device != dev and not m.locked:
                m.to(dev)
        return self

    def forward(self, input):
        weight = self.weight
        attrs = self.__dict__.get('_fp8_param_attrs')
        if attrs is not None and isinstance(weight, torch.Tensor) and not hasattr(weight, '_meta'):
            # a view of an FSDP flat parameter standing in for the fp32-viewed FP8 weight (msamp.fsdp.FsdpReplacer)
            for key, value in attrs['weight'].items():
                setattr(weight, key, value)
        return F.linear(input, weight, bias=self.bias)

    def extra_repr(self):
        return f'in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}'


class LinearReplacer:
    """Recursively replaces ``nn.Linear`` by FP8Linear, then syncs weights and registers the metas."""
    @staticmethod
    @torch.no_grad()
    def _build_fp8linear(linear, weight_qtype):
        if not isinstance(linear, torch.nn.Linear):
            raise TypeError('type of m must be torch.nn.Linear')
        src_dev = linear.weight.device
        device = default_device() if src_dev.type == 'cpu' else src_dev
        bias_dtype = linear.bias.dtype if linear.bias is not None else torch.float32
        fp8_linear = FP8Linear(
            linear.in_features, linear.out_features, use_bias=linear.bias is not None, weight_qtype=weight_qtype, bias_type=bias_dtype,
            device=device
        )
        if linear.bias is not None:
            fp8_linear.bias.data.copy_(linear.bias)
        w = linear.weight.detach().to(device)
        meta = ScalingMeta(weight_qtype, window_size=1, device=device)
        weight = w.cast(weight_qtype, meta=meta)
        if fp8_linear.weight.dtype != weight.dtype:
            raise ValueError(f'weight dtype mismatch: {fp8_linear.weight.dtype} vs {weight.dtype}')
        fp8_linear.weight.copy_(weight)
        fp8_linear.weight.requires_grad = linear.weight.requires_grad
        pairs = [(fp8_linear, linear), (fp8_linear.weight, linear.weight)]
        if linear.bias is not None:
            pairs.append((fp8_linear.bias, linear.bias))
        for new, old in pairs:
            _, custom = LinearReplacer._compare_attrs(type(old), old)
            for attr in custom:
                if not hasattr(new, attr):
                    setattr(new, attr, getattr(old, attr))
        return fp8_linear

    @staticmethod
    def _compare_attrs(x, y):
        """Names only ``x`` has and names only ``y`` has."""
        xs, ys = set(dir(x)), set(dir(y))
        return xs - ys, ys - xs

    @classmethod
    def _replace(cls, model, weight_qtype):
        if isinstance(model, torch.nn.Linear):
            if getattr(model, 'use_fp32_linear', False):
                return model
            return cls._build_fp8linear(model, weight_qtype)
        for name, child in list(model.named_children()):
            setattr(model, name, cls._replace(child, weight_qtype))
        return model

    @classmethod
    def replace(cls, model, weight_qtype=Dtypes.kfloat16, src_rank=0, group=None):
        """Convert ``model`` in place and return it.

        Besides the swap: broadcast the converted weights from ``src_rank``, tell DDP to ignore the
        FP8 parameters (they are reduced by msamp's own paths) and register all metas with ``model_state``.
        """
        model = cls._replace(model, weight_qtype)
        named = [(k, p) for k, p in model.named_parameters() if isinstance(p, ScalingParameter)]
        TensorDist.broadcast([p for _, p in named], src=src_rank, group=group)
        for k, p in named:
            p._param_name = k
        torch.nn.parallel.DistributedDataParallel._set_params_and_buffers_to_ignore_for_model(model, [k for k, _ in named])
        model_state.register_scaling_metas(model, group)
        return model
