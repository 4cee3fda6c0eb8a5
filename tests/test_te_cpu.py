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


def test_extension_helpers_with_fake_te_meta():
    """The TE-facing cast helpers give the same bytes for a plain tensor and for the ScalingTensor holding the same values
    when both use one scale (the property the reference checks in tests/te/test_extension.py:31-127), against a fake of
    TE's ``FP8TensorMeta`` (scale / scale_inv / amax_history indexed by tensor slot)."""
    import types

    from msamp.common.dtype import Dtypes
    from msamp.te.extension import TeExtensionOverrider, cast_to_fp8, fused_cast_transpose
    assert TeExtensionOverrider.installed is False    # Transformer Engine is not installed here; the helpers stand alone
    torch.manual_seed(0)
    x = torch.randn(16, 32)
    amax = x.abs().max()
    scale = torch.tensor(2.0**int(torch.floor(torch.log2(448.0 / amax))))
    slot = 1
    meta = types.SimpleNamespace(scale=torch.ones(3), scale_inv=torch.ones(3), amax_history=torch.zeros(4, 3))
    meta.scale[slot] = scale
    e4m3 = types.SimpleNamespace(name='kFloat8E4M3')
    out, out_t = fused_cast_transpose(x, meta, slot, e4m3)
    assert out.dtype == torch.uint8 and out.shape == (16, 32) and out_t.shape == (32, 16)
    assert torch.equal(out.t().contiguous(), out_t)
    assert abs(meta.amax_history[0][slot].item() - amax.item()) < 1e-6 and abs(meta.scale_inv[slot].item() - 1.0 / scale.item()) < 1e-9
    # the same values as an fp16 ScalingTensor: requantised from its meta, same scale, same bytes
    st = x.cast(Dtypes.kfloat16)
    meta2 = types.SimpleNamespace(scale=torch.ones(3), scale_inv=torch.ones(3), amax_history=torch.zeros(4, 3))
    out2, out2_t = fused_cast_transpose(st, meta2, slot, e4m3)
    back = out2.view(torch.float8_e4m3fn).float() * meta2.scale_inv[slot]
    assert (back - x).abs().max().item() <= 0.07 * amax.item()
    assert torch.equal(out2.reshape(16, 32).t().contiguous(), out2_t)
    single = cast_to_fp8(x, meta, slot, e4m3)
    assert torch.equal(single, out)
    buf = torch.empty(16, 32, dtype=torch.uint8)
    assert cast_to_fp8(x, meta, slot, e4m3, out=buf) is None and torch.equal(buf, out)
    e5m2 = types.SimpleNamespace(name='kFloat8E5M2')
    assert cast_to_fp8(x, meta, slot, e5m2).dtype == torch.uint8
