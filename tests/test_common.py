"""CPU unit tests of the core layer: dtypes, floating ranges, ScalingMeta, casts, ScalingTensor, hooks, torch patches."""
import pickle

import pytest
import torch

import msamp    # noqa: F401
from msamp.common.dtype import Dtypes, Floating, QType
from msamp.common.tensor import HookManager, ScalingMeta, ScalingTensor, TypeCast
from msamp.common.utils import DistUtil, LazyImport, logger

E4, E5, F16, BF16, F32 = Dtypes.kfloat8_e4m3, Dtypes.kfloat8_e5m2, Dtypes.kfloat16, Dtypes.kbfloat16, Dtypes.kfloat32


def test_dtypes_and_qtypes():
    assert torch.fp8e4m3 is torch.uint8 and torch.fp8e5m2 is torch.int8
    assert [int(q) for q in (Dtypes.kbyte, Dtypes.kint32, F32, F16, BF16, E4, E5)] == list(range(7))
    assert Dtypes.is_fp8_qtype(E4) and Dtypes.is_fp8_qtype(E5) and not Dtypes.is_fp8_qtype(F16)
    assert Dtypes.get_dtype_from_qtype(E4) is torch.uint8 and Dtypes.get_dtype_from_qtype(E5) is torch.uint8
    assert Dtypes.get_dtype_from_qtype(F16) is torch.float16
    assert Dtypes.dtype_to_qtype[torch.int8] == E5 and Dtypes.qtype_to_dtype[E4] is torch.uint8
    assert hash(QType('x', 5)) == 5 and QType('kFloat8E4M3', 5) == E4
    assert torch.randn(2).qtype == F32 and torch.randn(2).half().qtype == F16


def test_floating_max_values():
    assert Floating.qfp_max[E4] == 448.0 and Floating.qfp_max[E5] == 57344.0 and Floating.qfp_max[F16] == 65504.0
    assert Floating.fp_maxs[torch.bfloat16] == torch.finfo(torch.bfloat16).max
    assert Floating.fp_maxs[torch.float32] == torch.finfo(torch.float32).max
    assert Floating._get_fp_max(4, 3, inf_existed=True) == 240.0


def test_scale_rule_golden():
    one = torch.ones(())
    f = lambda a: ScalingMeta.compute_scaling_factor(torch.tensor(a), one, 448.0, 0).item()    # noqa: E731
    assert f(10.0) == 32.0 and f(1e4) == 1 / 32 and f(0.0) == 1.0 and f(448.0) == 1.0
    assert f(float('inf')) == 1.0 and f(float('nan')) == 1.0
    assert ScalingMeta.compute_scaling_factor(torch.tensor(10.0), one, 448.0, 2).item() == 8.0


def test_meta_warmup_and_context():
    m = ScalingMeta(E4, window_size=4)
    assert m.is_warmup() and m.is_in_time_scaling()
    m.amax_counter += 4
    assert not m.is_warmup() and not m.is_in_time_scaling()
    m1 = ScalingMeta(E4, window_size=1)
    m1.amax_counter += 10
    assert m1.is_in_time_scaling()
    with ScalingMeta.in_time_scaling_context(False):
        assert not m1.is_in_time_scaling()
    assert m1.is_in_time_scaling()
    c = m.clone()
    c.scale.fill_(3)
    assert m.scale.item() == 1 and c.window_size == 4
    assert 'ScalingMeta' in repr(m)


@pytest.mark.parametrize('q', [E4, E5])
def test_fp8_cast_roundtrip_and_saturation(q):
    x = torch.randn(1000) * 5
    t = x.cast(q)
    assert t.value.dtype == torch.uint8 and t.meta.amax[0].item() == x.abs().max().item()
    rel = 0.07 if q == E4 else 0.13
    assert ((t.float() - x).abs() <= rel * x.abs() + 1e-2).all()
    assert t.meta.scale.item() * t.meta.scale_inv.item() == 1.0
    # explicit scale that overflows: values saturate at the format maximum instead of becoming inf/nan
    meta = ScalingMeta(q, scale=torch.tensor(1e6), window_size=16)
    meta.amax_counter += 16    # delayed scaling: keep the given scale
    y = TypeCast.cast_to_fp8(torch.tensor([1.0, -1.0, 0.0]), meta)
    back = TypeCast.cast_from_fp8(y, meta, F32) * 1e6
    assert back.tolist() == [Floating.qfp_max[q], -Floating.qfp_max[q], 0.0]
    assert meta.amax[0].item() == 1.0    # recorded for later


def test_nan_inf_reach_amax():
    x = torch.randn(16)
    x[3] = float('nan')
    t = x.cast(E4)
    assert t.has_inf_or_nan() and t.meta.scale.item() == 1.0
    x[3] = float('inf')
    assert x.cast(E5).has_inf_or_nan()
    assert not torch.randn(4).cast(E4).has_inf_or_nan()
    assert bool(t.isnan()[3]) and not bool(t.isnan()[0])


def test_cast_matrix_between_qtypes():
    x = torch.randn(64, 32)
    for q1 in (E4, E5, F16, BF16, F32):
        a = x.cast(q1)
        for q2 in (E4, E5, F16, BF16, F32):
            b = a.cast(q2)
            assert b.qtype == q2
            assert torch.allclose(b.float(), x, rtol=0.13, atol=0.13)
    assert a.cast(a.qtype) is a
    c = x.cast(F16)
    c.cast_(E4)
    assert c.qtype == E4 and c.dtype == torch.uint8


def test_fused_cast_transpose_and_fp8_transpose():
    x = torch.randn(24, 40)
    a, at = x.fused_cast_transpose(E5)
    assert torch.equal(a.value.t(), at.value) and a.meta is at.meta
    assert torch.equal(a.fp8_transpose().value, at.value)
    with pytest.raises(TypeError):
        x.fused_cast_transpose(F16)
    with pytest.raises(TypeError):
        x.cast(F16).fp8_transpose()


def test_mul_div_touch_only_scale_inv():
    t = torch.randn(10).cast(E4)
    v, ref = t.value.clone(), t.float()
    t.mul_(2.0)
    assert torch.equal(t.value, v) and torch.equal(t.float(), ref * 2)
    t.div_(torch.tensor(4.0))
    assert torch.equal(t.float(), ref / 2)
    with pytest.raises(ValueError):
        t.mul_(torch.ones(2))


def test_tensor_surface():
    x = torch.randn(4, 6)
    t = x.cast(E4)
    assert t.shape == (4, 6) and t.size(0) == 4 and t.numel() == 24 and len(t) == 4 and t.dim() == 2
    assert t.t().shape == (6, 4) and t.flatten().shape == (24, ) and t.contiguous().value.is_contiguous()
    assert not t.is_floating_point() and not torch.is_floating_point(t) and torch.is_floating_point(x)
    assert t.is_leaf and t.grad_fn is None and t.grad is None and not t.is_cuda
    assert t.to(torch.float16).dtype == torch.float16 and t.half().dtype == torch.float16 and t.bfloat16().dtype == torch.bfloat16
    with pytest.raises(TypeError):
        t.to(torch.int32)
    with pytest.raises(TypeError):
        t.to(torch.float32, dtype=torch.float32)
    assert torch.equal(t.abs().value, t.value & 0x7F)
    assert t.max().item() == t.float().max().item() and t.min().item() == t.float().min().item()
    c = t.clone()
    c.zero_()
    assert t.value.any() and not c.value.any()
    d = torch.zeros(4, 6).cast(E4)
    d.copy_(t)
    assert torch.equal(d.value, t.value) and d.meta.scale.item() == t.meta.scale.item()
    with pytest.raises(TypeError):
        d.copy_(x)
    with pytest.raises(TypeError):
        ScalingTensor(x, ScalingMeta(E4))
    assert torch.zeros_like(t).dtype == torch.uint8 and torch.ones_like(t).shape == t.shape
    assert torch.overrides.is_tensor_like(t)
    assert t.pad((0, 2)).shape == (4, 8) and 'ScalingTensor' in repr(t)
    assert t.type() == 'msamp.common.tensor.tensor.ScalingTensor'


def test_locked_meta_blocks_replacement():
    t = torch.randn(4).cast(E4)
    other = torch.randn(4).cast(E4)
    t.meta.locked = True
    with pytest.raises(ValueError):
        t.data = other
    t.data = ScalingTensor(other.value, t.meta)


def test_pickle_layout_is_the_reference_layout():
    t = torch.randn(8).cast(E4)
    blob = pickle.dumps(t)
    assert b'msamp.common.tensor.tensor' in blob and b'msamp.common.tensor.meta' in blob and b'msamp.common.dtype.dtypes' in blob
    u = pickle.loads(blob)
    assert set(u.__dict__) >= {'value', 'meta', '_grad', '_backward_post_hooks', '_requires_grad'}
    assert set(u.meta.__dict__) >= {'qtype', 'scale', 'scale_inv', 'amax', 'amax_counter', 'window_size', 'group', 'locked'}
    assert set(u._backward_post_hooks.__dict__) == {'hooks', 'history_counter'}
    assert torch.equal(u.float(), t.float())


def test_hook_manager():
    seen = []
    hm = HookManager()
    h1 = hm.register_hook(lambda mod, inp, out: seen.append((inp[0], out)))
    h2 = hm.register_hook(lambda mod, inp, out: seen.append((inp[0], out)))
    x = torch.randn(2, 3)
    hm(x)
    assert len(seen) == 2 and all(a is x and b is x for a, b in seen)
    h1.remove()
    h2.remove()
    seen.clear()
    hm(x)
    assert not seen
    t = torch.randn(3).cast(E4)
    t.register_backward_post_hook(lambda *a, **k: seen.append('g'))
    t.backward_grad_update(torch.ones(3))
    assert seen == ['g'] and t.grad is not None


def test_grad_scaler_unscale_wrapper():
    g1 = torch.full((4, ), 8.0)
    st = torch.randn(4).cast(E4)
    ref = st.float()
    found = torch.zeros(1)
    torch._amp_foreach_non_finite_check_and_unscale_([g1, st], found, torch.tensor(0.5))
    assert torch.equal(g1, torch.full((4, ), 4.0)) and torch.equal(st.float(), ref * 0.5) and found.item() == 0
    bad = torch.tensor([1.0, float('inf')]).cast(E4)
    torch._amp_foreach_non_finite_check_and_unscale_([bad], found, torch.tensor(1.0))
    assert found.item() == 1


def test_utils():
    assert DistUtil.get_world_size() == 1 and DistUtil.get_rank() == 0 and DistUtil.is_main_process()
    lazy = LazyImport('math')
    assert lazy.sqrt(4.0) == 2.0
    with pytest.raises(ValueError):
        logger.log_and_raise(ValueError, 'boom %d', 1)
