"""TE-style modules and replacer (Transformer Engine itself is optional and absent here)."""
import torch

import msamp
from msamp.common.utils import TransformerEngineWrapper
from msamp.common.dtype import Dtypes
from msamp.nn import ScalingParameter
from msamp.te import MSAMPLayerNormLinear, MSAMPLayerNormMLP, MSAMPLinear, MSAMPTransformerLayer, TeReplacer, te_available
from msamp.te.extension import cast_if_needed


class Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.a = MSAMPLinear(32, 64)
        self.b = MSAMPLayerNormLinear(64, 64)
        self.c = MSAMPLayerNormMLP(64, 128)

    def forward(self, x):
        return self.c(self.b(self.a(x)))


def test_replacer_counts_and_training():
    torch.manual_seed(0)
    model = Net()
    model, opt = msamp.initialize(model, None, 'O2', use_te=True)
    for g in opt.param_groups:
        g['lr'] = 1e-2
    scaling = [p for p in model.parameters() if isinstance(p, ScalingParameter)]
    assert len(scaling) == 4    # three modules, four FP8 weights
    assert sorted(model._ddp_params_and_buffers_to_ignore) == ['a.weight', 'b.weight', 'c.fc1_weight', 'c.fc2_weight']
    from msamp.nn import model_state
    assert model_state.flattened_scaling_metas['input']['scales'].numel() == 4
    x, y = torch.randn(16, 32), torch.randn(16, 64)
    losses = []
    for _ in range(10):
        opt.zero_grad()
        loss = ((model(x) - y)**2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
    assert TeReplacer.module_weight_names[MSAMPLayerNormMLP] == ['fc1_weight', 'fc2_weight']
    assert te_available() in (True, False)


def test_transformer_layer_shapes():
    layer = MSAMPTransformerLayer(64, 256, 4)
    x = torch.randn(10, 2, 64, requires_grad=True)
    y = layer(x)
    assert y.shape == x.shape
    y.sum().backward()
    assert x.grad is not None and layer.proj.weight.grad is not None


def test_wrapper_matches_kernels():
    x = torch.randn(8, 16)
    scale, amax, sinv = torch.tensor(4.0), torch.zeros(()), torch.ones(())
    q = TransformerEngineWrapper.cast_to_fp8(x, scale, amax, sinv, Dtypes.kfloat8_e4m3)
    assert q.dtype == torch.uint8 and amax.item() == x.abs().max().item() and sinv.item() == 0.25
    back = TransformerEngineWrapper.cast_from_fp8(q, sinv, Dtypes.kfloat8_e4m3, Dtypes.kfloat32)
    assert (back - x).abs().max() < 0.3
    a = torch.ones(4, 16).cast(Dtypes.kfloat8_e4m3)
    b = torch.ones(8, 16).cast(Dtypes.kfloat8_e4m3)
    D = torch.empty(8, 4)
    TransformerEngineWrapper.te_gemm(a.value, a.meta.scale_inv, a.qtype, True, b.value, b.meta.scale_inv, b.qtype, False, D, None,
                                     Dtypes.kfloat32, None, torch.empty(0), Dtypes.kfloat32, None, False, None, 0, False, False)
    assert (D == 16).all()
    assert TransformerEngineWrapper._to_te_dtype(Dtypes.kfloat8_e5m2) == 'kFloat8E5M2'
    st = torch.randn(4).cast(Dtypes.kfloat16)
    assert cast_if_needed(st, torch.float32) is st and cast_if_needed(torch.ones(2), torch.float16).dtype == torch.float16
