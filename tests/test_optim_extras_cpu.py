"""Loss scaling policy, overflow detection, the single-process O3 optimizer and FSDPAdamW on flat FP8 parameters."""
import torch

import msamp
from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingMeta, ScalingTensor


def test_dynamic_loss_scaler_policy():
    from msamp.deepspeed.runtime.fp8.loss_scaler import DynamicLossScaler, LossScaler
    s = LossScaler(128.0)
    s.update_scale(True)
    assert s.loss_scale == 128.0 and not s.dynamic
    d = DynamicLossScaler(init_scale=2**10, scale_window=4, hysteresis=2, min_scale=1.0)
    d.update_scale(True)    # first overflow only uses up the hysteresis
    assert d.cur_scale == 2**10
    d.update_scale(True)
    assert d.cur_scale == 2**9
    for _ in range(4):
        d.update_scale(False)
    assert d.cur_scale == 2**10    # a clean window doubles again
    tiny = DynamicLossScaler(init_scale=2.0, hysteresis=1, min_scale=1.0)
    for _ in range(5):
        tiny.update_scale(True)
    assert tiny.cur_scale == 1.0
    e = DynamicLossScaler()
    e.load_state_dict(d.state_dict())
    assert e.state_dict() == d.state_dict()


def test_overflow_check_understands_scaling_tensors():
    from msamp.deepspeed.runtime.utils import MSAMPCheckOverflow
    chk = MSAMPCheckOverflow()
    a, b = torch.nn.Parameter(torch.ones(4)), torch.nn.Parameter(torch.ones(4))
    a.grad, b.grad = torch.ones(4), torch.ones(4)
    assert not chk.check([a, b])
    b.grad = torch.tensor([1.0, float('inf'), 0.0, 0.0])
    assert chk.check([a, b])
    g = torch.randn(8).cast(Dtypes.kfloat8_e4m3)
    assert not chk.has_overflow([g, None])
    g.meta.amax[0] = float('nan')
    assert chk.has_overflow([g])


def test_o3_master_optimizer_single_process():
    from msamp.nn import FP8Linear
    from msamp.optim.master import FP8MasterOptimizer
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 16))
    opt = torch.optim.AdamW(model.parameters(), lr=5e-3)
    model, opt = msamp.initialize(model, opt, 'O3')
    assert isinstance(opt, FP8MasterOptimizer) and isinstance(model[0], FP8Linear)
    assert model[0].weight.qtype == Dtypes.kfloat8_e4m3    # O3 keeps the model weights themselves in FP8
    x, y = torch.randn(32, 16), torch.randn(32, 16)
    losses = []
    for _ in range(30):
        opt.zero_grad()
        loss = ((model(x) - y)**2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.8 * losses[0], losses
    sd = opt.state_dict()
    opt.load_state_dict(sd)
    assert len(opt.param_groups) >= 1 and opt.state is not None


def test_fsdp_adamw_updates_flat_fp8_parameter():
    from msamp.optim import FSDPAdamW
    torch.manual_seed(0)
    w = torch.randn(8, 16) * 0.1
    w8 = w.cast(Dtypes.kfloat8_e4m3)
    flat = torch.nn.Parameter(w8.value.reshape(-1).view(torch.float32).clone())    # FP8 bytes viewed as fp32, as in an FSDP flat parameter
    flat._meta = w8.meta
    flat._grad_meta = ScalingMeta(Dtypes.kfloat8_e4m3)
    bias = torch.nn.Parameter(torch.zeros(8))
    opt = FSDPAdamW([flat, bias], lr=1e-2, weight_decay=0.0)
    before = ScalingTensor(flat.detach().view(torch.uint8).clone().view(8, 16), flat._meta.clone()).float()
    g = torch.ones(8, 16).cast(Dtypes.kfloat8_e4m3, meta=flat._grad_meta)
    flat.grad = g.value.reshape(-1).view(torch.float32).clone()
    bias.grad = torch.ones(8)
    opt.step()
    after = ScalingTensor(flat.detach().view(torch.uint8).view(8, 16), flat._meta).float()
    # a positive gradient moves every weight down by about lr
    delta = (before - after)
    assert delta.mean().item() > 0.005 and delta.mean().item() < 0.02
    assert torch.allclose(bias.detach(), torch.full((8, ), -1e-2), atol=1e-4)
    opt.zero_grad(set_to_none=True)
    assert flat.grad is None


def test_scale_histogram_reports_registered_layers():
    from msamp.nn import LinearReplacer, model_state
    from msamp.utils import StepMetrics
    model = LinearReplacer.replace(torch.nn.Sequential(torch.nn.Linear(16, 16), torch.nn.Linear(16, 16)))
    model_state.register_scaling_metas(model)
    h = StepMetrics.scale_histogram()
    assert set(h) >= {'input', 'wgrad', 'ograd'} and h['input']['layers'] == 2
    model_state.clear() if hasattr(model_state, 'clear') else None
