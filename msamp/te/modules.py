"""Fused transformer modules in the shape of Transformer Engine's ``Linear``, ``LayerNormLinear``, ``LayerNormMLP``.

The reference subclasses TE's modules and wraps their autograd functions so that ScalingTensor weights can
be saved for backward and the weight gradient is delivered through ``backward_grad_update``
(msamp/te/modules.py:20-290).  These classes provide the same modules on msamp's own kernels
(LayerNorm → FP8 cast → tcgen05 GEMM → GeLU), so ``use_te=True`` works whether or not Transformer
Engine is installed; when it is, ``TeReplacer`` converts TE modules into these, copying their weights
(parameter names ``weight``, ``layer_norm_weight``, ``layer_norm_bias``, ``fc1_weight``, ``fc2_weight``… follow TE).
"""
import torch
import torch.nn.functional as F

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingMeta
from msamp.nn.module import ScalingModule
from msamp.nn import fused_layers as FL
from msamp.nn.parameter import ScalingParameter
from msamp.ops import nn as K

E4M3, E5M2 = Dtypes.kfloat8_e4m3, Dtypes.kfloat8_e5m2


def te_available():
    """True if ``transformer_engine.pytorch`` can be imported."""
    try:
        import transformer_engine.pytorch    # noqa: F401
        return True
    except Exception:
        return False


def _metas(device):
    return dict(
        input=ScalingMeta(E4M3, window_size=16, device=device),
        wgrad=ScalingMeta(E4M3, window_size=1, device=device),
        ograd=ScalingMeta(E5M2, window_size=16, device=device),
    )


def _weight(out_f, in_f, device, std=0.02):
    w = torch.empty(out_f, in_f, device=device).normal_(0.0, std)
    return ScalingParameter(w.cast(Dtypes.kfloat16, meta=ScalingMeta(Dtypes.kfloat16, window_size=1, device=w.device)))


class MSAMPLinear(ScalingModule):
    """``te.Linear``: FP8 linear with a ScalingParameter ``weight`` and optional ``bias``."""
    is_msamp_module = True

    def __init__(self, in_features, out_features, bias=True, device=None, **unused):
        super().__init__()
        dev = torch.device(device) if device is not None else torch.device('cpu')
        self.in_features, self.out_features = in_features, out_features
        self.weight = _weight(out_features, in_features, dev)
        self.bias = torch.nn.Parameter(torch.zeros(out_features, device=dev)) if bias else None
        self.scaling_metas = _metas(dev)
        self.weight._scaling_metas = self.scaling_metas

    def forward(self, x):
        return F.linear(x, self.weight, self.bias)


class MSAMPLayerNormLinear(ScalingModule):
    """``te.LayerNormLinear``: LayerNorm followed by an FP8 linear."""
    is_msamp_module = True

    def __init__(self, in_features, out_features, eps=1e-5, bias=True, device=None, return_layernorm_output=False, **unused):
        super().__init__()
        dev = torch.device(device) if device is not None else torch.device('cpu')
        self.in_features, self.out_features, self.eps = in_features, out_features, eps
        self.return_layernorm_output = return_layernorm_output
        self.layer_norm_weight = torch.nn.Parameter(torch.ones(in_features, device=dev))
        self.layer_norm_bias = torch.nn.Parameter(torch.zeros(in_features, device=dev))
        self.weight = _weight(out_features, in_features, dev)
        self.bias = torch.nn.Parameter(torch.zeros(out_features, device=dev)) if bias else None
        self.scaling_metas = _metas(dev)
        self.weight._scaling_metas = self.scaling_metas

    def _views(self):
        return (FL.ModuleView(self.layer_norm_weight, self.layer_norm_bias, self.eps),
                FL.ModuleView(self.weight, self.bias, scaling_metas=self.scaling_metas))

    def forward(self, x):
        if not self.return_layernorm_output and isinstance(self.weight, ScalingParameter) and x.dim() == 2:
            ln, lin = self._views()
            return FL.ln_linear(x, ln, lin)    # LayerNorm emits e4m3 directly: its output is never stored in 16 bits
        ln = K.layer_norm(x, self.layer_norm_weight, self.layer_norm_bias, self.eps)
        out = F.linear(ln, self.weight, self.bias)
        return (out, ln) if self.return_layernorm_output else out


class MSAMPLayerNormMLP(ScalingModule):
    """``te.LayerNormMLP``: LayerNorm → FP8 linear → GeLU → FP8 linear."""
    is_msamp_module = True

    def __init__(self, hidden_size, ffn_hidden_size, eps=1e-5, bias=True, device=None, **unused):
        super().__init__()
        dev = torch.device(device) if device is not None else torch.device('cpu')
        self.hidden_size, self.ffn_hidden_size, self.eps = hidden_size, ffn_hidden_size, eps
        self.layer_norm_weight = torch.nn.Parameter(torch.ones(hidden_size, device=dev))
        self.layer_norm_bias = torch.nn.Parameter(torch.zeros(hidden_size, device=dev))
        self.fc1_weight = _weight(ffn_hidden_size, hidden_size, dev)
        self.fc2_weight = _weight(hidden_size, ffn_hidden_size, dev)
        self.fc1_bias = torch.nn.Parameter(torch.zeros(ffn_hidden_size, device=dev)) if bias else None
        self.fc2_bias = torch.nn.Parameter(torch.zeros(hidden_size, device=dev)) if bias else None
        self.fc1_metas, self.fc2_metas = _metas(dev), _metas(dev)
        self.scaling_metas = self.fc1_metas
        self.fc1_weight._scaling_metas = self.fc1_metas
        self.fc2_weight._scaling_metas = self.fc2_metas
        self._second = _MetaHolder(self.fc2_metas)

    def _views(self):
        return (FL.ModuleView(self.layer_norm_weight, self.layer_norm_bias, self.eps),
                FL.ModuleView(self.fc1_weight, self.fc1_bias, scaling_metas=self.fc1_metas),
                FL.ModuleView(self.fc2_weight, self.fc2_bias, scaling_metas=self.fc2_metas))

    def forward(self, x, residual=False):
        """``fc2(gelu(fc1(layer_norm(x))))``; ``residual=True`` adds ``x`` in the epilogue of the fc2 GEMM."""
        if isinstance(self.fc1_weight, ScalingParameter) and isinstance(self.fc2_weight, ScalingParameter) and x.dim() == 2:
            ln, fc1, fc2 = self._views()
            return FL.mlp_sublayer(x, ln, fc1, fc2, residual=residual)
        ln = K.layer_norm(x, self.layer_norm_weight, self.layer_norm_bias, self.eps)
        h = K.gelu(F.linear(ln, self.fc1_weight, self.fc1_bias))
        out = F.linear(h, self.fc2_weight, self.fc2_bias)
        return x + out if residual else out


class _MetaHolder(torch.nn.Module):
    """Carries a second set of scaling metas so that ``model_state.register_scaling_metas`` finds both GEMMs of an MLP."""
    def __init__(self, metas):
        super().__init__()
        self.scaling_metas = metas


class MSAMPTransformerLayer(torch.nn.Module):
    """``te.TransformerLayer`` (pre-LayerNorm encoder/decoder block with causal or full self-attention)."""
    def __init__(self, hidden_size, ffn_hidden_size, num_attention_heads, layernorm_epsilon=1e-5, self_attn_mask_type='causal',
                 device=None, **unused):
        super().__init__()
        self.num_heads, self.head_dim = num_attention_heads, hidden_size // num_attention_heads
        self.causal = self_attn_mask_type == 'causal'
        self.layernorm_qkv = MSAMPLayerNormLinear(hidden_size, 3 * hidden_size, eps=layernorm_epsilon, device=device)
        self.proj = MSAMPLinear(hidden_size, hidden_size, device=device)
        self.layernorm_mlp = MSAMPLayerNormMLP(hidden_size, ffn_hidden_size, eps=layernorm_epsilon, device=device)

    def forward(self, hidden_states, attention_mask=None):
        # hidden_states: [seq, batch, hidden] as in TE
        s, b, h = hidden_states.shape
        x = hidden_states.transpose(0, 1).contiguous()
        fused_attention = (not x.is_cuda) or (x.dtype == torch.bfloat16 and self.head_dim in (64, 128))
        if fused_attention and isinstance(self.layernorm_qkv.weight, ScalingParameter) and isinstance(self.proj.weight, ScalingParameter):
            # both halves of the block as fused sublayers (msamp.nn.fused_layers)
            ln, qkv_lin = self.layernorm_qkv._views()
            x2 = FL.attention_sublayer(x.view(b * s, h), ln, qkv_lin, self.proj, b, s, self.num_heads, causal=self.causal)
            x2 = self.layernorm_mlp(x2, residual=True)
            return x2.view(b, s, h).transpose(0, 1).contiguous()
        qkv = self.layernorm_qkv(x.view(b * s, h)).view(b, s, 3, self.num_heads, self.head_dim)
        o = K.attention_qkv(qkv, causal=self.causal) if qkv.is_cuda and qkv.dtype == torch.bfloat16 and self.head_dim in (64, 128) else \
            K.attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal=self.causal) if not qkv.is_cuda else _sdpa(qkv, self.causal)
        x = x.view(b * s, h) + self.proj(o.reshape(b * s, h))
        x = x + self.layernorm_mlp(x)
        return x.view(b, s, h).transpose(0, 1).contiguous()


def _sdpa(qkv, causal):
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    return F.scaled_dot_product_attention(q, k, v, is_causal=causal).permute(0, 2, 1, 3)
