"""GPU numerics: every native kernel against a plain PyTorch fp32 reference (or the CPU emulation, bit for bit)."""
import math

import pytest
import torch

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingMeta
from msamp.ops import arith, cast, gemm, native, reduce
from msamp.ops import nn as K

pytestmark = pytest.mark.gpu
E4, E5 = Dtypes.kfloat8_e4m3, Dtypes.kfloat8_e5m2
F8 = Dtypes.qtype_to_float8
DEV = 'cuda'


def _status_ok():
    torch.cuda.synchronize()
    assert native.device_status() == 0


def test_amax_and_nan():
    x = torch.randn(1000, 333, device=DEV, dtype=torch.bfloat16)
    assert cast.amax(x).item() == x.float().abs().max().item()
    x[5, 7] = float('nan')
    assert cast.amax(x).item() == float('inf')
    assert cast.amax(torch.zeros(0, device=DEV)).item() == 0


@pytest.mark.parametrize('dt', [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize('q', [E4, E5])
def test_cast_bit_exact(dt, q):
    for n in (1, 7, 4096, 1000003):
        x = (torch.randn(n, device=DEV) * 3).to(dt)
        x[0] = 1e6    # saturates
        s = torch.tensor(16.0, device=DEV)
        am = torch.zeros((), device=DEV)
        si = torch.zeros((), device=DEV)
        y = cast.cast_to_fp8(x, q, s, am, scale_inv_out=si)
        ref = cast.cast_to_fp8(x.cpu(), q, s.cpu())
        assert torch.equal(y.cpu(), ref)
        assert am.item() == x.float().abs().max().item() and si.item() == 1 / 16
        back = cast.cast_from_fp8(y, q, si, dt)
        assert torch.equal(back.cpu(), cast.cast_from_fp8(ref, q, si.cpu(), dt))
    # unaligned views take the scalar path
    x = torch.randn(1001, device=DEV, dtype=torch.bfloat16)[1:]
    y = cast.cast_to_fp8(x, q, torch.tensor(4.0, device=DEV))
    assert torch.equal(y.cpu(), cast.cast_to_fp8(x.cpu(), q, torch.tensor(4.0)))


@pytest.mark.parametrize('shape', [(64, 64), (128, 256), (100, 72), (1024, 4096), (33, 17), (16, 8)])
def test_cast_transpose(shape):
    for dt in (torch.bfloat16, torch.float32):
        x = torch.randn(*shape, device=DEV, dtype=dt)
        s = torch.tensor(8.0, device=DEV)
        am = torch.zeros((), device=DEV)
        o, ot = cast.cast_transpose_fp8(x, E4, s, am)
        ref = cast.cast_to_fp8(x.cpu(), E4, s.cpu())
        assert torch.equal(o.cpu(), ref) and torch.equal(ot.cpu(), ref.t().contiguous())
        assert torch.equal(cast.transpose_fp8(o).cpu(), ref.t().contiguous())
        assert am.item() == x.float().abs().max().item()
        _, ot2 = cast.cast_transpose_fp8(x, E5, s, need_rowmajor=False)
        assert torch.equal(ot2.cpu(), cast.cast_to_fp8(x.cpu(), E5, s.cpu()).t().contiguous())
        # column sums from the same pass (added to the buffer)
        cs = torch.ones(shape[1], device=DEV)
        o3, ot3 = cast.cast_transpose_fp8(x, E4, s, am, colsum_out=cs)
        assert torch.equal(o3, o) and torch.equal(ot3, ot)
        want = 1.0 + x.double().sum(0)
        assert (cs.double() - want).abs().max().item() <= 1e-4 * max(1.0, x.float().abs().sum(0).max().item())


def test_in_time_scale_and_windows():
    x = torch.randn(4096, device=DEV) * 10
    am, sc, si = torch.zeros((), device=DEV), torch.ones((), device=DEV), torch.ones((), device=DEV)
    cast.amax_and_scale(x, am, sc, si, E4)
    ref = ScalingMeta.compute_scaling_factor(x.abs().max().cpu(), torch.ones(()), 448.0, 0)
    assert sc.item() == ref.item() and si.item() == 1 / ref.item()
    # golden values of the scale rule
    for amax, want in ((10.0, 32.0), (1e4, 1 / 32), (0.0, 1.0)):
        a = torch.tensor([amax], device=DEV)
        s, i = torch.ones(1, device=DEV), torch.ones(1, device=DEV)
        cast.update_scales(a, s, i, E4)
        assert s.item() == want
    # window roll matches the CPU definition
    amaxs = torch.rand(7, 16, device=DEV) * 100
    amaxs[2, 0] = float('inf')
    scales = torch.ones(7, device=DEV)
    a2, s2 = amaxs.cpu().clone(), scales.cpu().clone()
    bad = torch.zeros(7, dtype=torch.int32, device=DEV)
    cast.roll_windows(amaxs, scales, E4, bad_out=bad)
    cast.roll_windows(a2, s2, E4)
    assert torch.equal(amaxs.cpu(), a2) and torch.equal(scales.cpu(), s2)
    assert bad.cpu().tolist() == [0, 0, 1, 0, 0, 0, 0]


def _mk(m, k, q, scale=32.0):
    x = torch.randn(m, k, device=DEV)
    s = torch.tensor(scale, device=DEV)
    return cast.cast_to_fp8(x, q, s), torch.tensor(1 / scale, device=DEV)


def test_gemm_all_ones_exact():
    a = torch.full((128, 128), 0x38, dtype=torch.uint8, device=DEV)    # 1.0 in e4m3
    one = torch.ones((), device=DEV)
    d = gemm.gemm_fp8(a, E4, one, a.clone(), E4, one, torch.float32)
    assert (d == 128).all()
    _status_ok()


@pytest.mark.parametrize('mnk', [(128, 128, 128), (256, 512, 1024), (128, 256, 4096), (100, 72, 48), (1000, 520, 272), (4096, 4096, 2048),
                                 (2048, 50304, 256), (1, 16, 16), (300, 8, 40)])
@pytest.mark.parametrize('qa', [E4, E5])
def test_gemm_vs_fp32(mnk, qa):
    m, n, k = mnk
    a, sia = _mk(m, k, qa)
    b, sib = _mk(n, k, E4)
    bias = torch.randn(n, device=DEV)
    ref = (a.view(F8[qa]).float() @ b.view(F8[E4]).float().t()) * (sia * sib)
    sc = ref.abs().max().item() + 1e-6
    d32 = gemm.gemm_fp8(a, qa, sia, b, E4, sib, torch.float32)
    assert (d32 - ref).abs().max().item() <= 1e-4 * sc + 1e-4
    am = torch.zeros((), device=DEV)
    d16 = gemm.gemm_fp8(a, qa, sia, b, E4, sib, torch.bfloat16, bias=bias, amax_out=am)
    assert (d16.float() - (ref + bias)).abs().max().item() <= 1e-2 * (sc + 4)
    assert abs(am.item() - d16.float().abs().max().item()) <= 1e-2 * (sc + 4)
    acc = gemm.gemm_fp8(a, qa, sia, b, E4, sib, torch.float32, accumulate=True, out=d32.clone())
    assert (acc - 2 * ref).abs().max().item() <= 2e-4 * sc + 1e-4
    dh = gemm.gemm_fp8(a, qa, sia, b, E4, sib, torch.float16, bias=bias.half())
    assert (dh.float() - (ref + bias.half().float())).abs().max().item() <= 2e-3 * (sc + 4)
    _status_ok()


def test_gemm_strided_and_capped():
    a, sia = _mk(512, 1024, E4)
    b, sib = _mk(384, 1024, E4)
    ref = (a.view(F8[E4]).float() @ b.view(F8[E4]).float().t()) * (sia * sib)
    out = torch.zeros(512, 1000, device=DEV)
    gemm.gemm_fp8(a[:, :512], E4, sia, b[:, :512], E4, sib, torch.float32, out=out[:, 8:392])
    ref2 = (a[:, :512].view(F8[E4]).float() @ b[:, :512].view(F8[E4]).float().t()) * (sia * sib)
    assert (out[:, 8:392] - ref2).abs().max().item() < 1e-3 and out[:, :8].abs().max().item() == 0
    d = gemm.gemm_fp8(a, E4, sia, b, E4, sib, torch.float32, max_ctas=3)
    assert (d - ref).abs().max().item() < 1e-3
    _status_ok()


@pytest.mark.parametrize('shape', [(256, 512), (1000, 264), (8192, 4096), (3, 8)])
def test_cast_colsum_gelu_rescale(shape):
    """Options of the plain cast: column sums of the input, GeLU before quantising, re-quantising a scaled tensor."""
    x = (torch.randn(*shape, device=DEV) * 3).bfloat16()
    s = torch.tensor(4.0, device=DEV)
    am, si = torch.zeros((), device=DEV), torch.zeros((), device=DEV)
    cs = torch.zeros(shape[1], device=DEV)
    out = cast.cast_to_fp8(x, E5, s, am, scale_inv_out=si, colsum_out=cs)
    assert torch.equal(out.cpu(), cast.cast_to_fp8(x.cpu(), E5, s.cpu()))
    assert am.item() == x.float().abs().max().item() and si.item() == 0.25
    ref = x.float().sum(0)
    assert (cs - ref).abs().max().item() <= 1e-3 * (ref.abs().max().item() + shape[0] ** 0.5)
    # GeLU folded into the cast == GeLU kernel followed by the cast
    am2 = torch.zeros((), device=DEV)
    fused = cast.cast_to_fp8(x, E4, s, am2, act='gelu')
    g = K.gelu(x)
    assert torch.equal(fused, cast.cast_to_fp8(g, E4, s)) and am2.item() == g.float().abs().max().item()
    # scaled 16-bit tensor (x0 * s_old) -> e4m3 with the scale implied by amax(x0)
    s_old = 8.0
    x0 = torch.randn(*shape, device=DEV)
    xs = (x0 * s_old).half()
    amax0 = (xs.float() / s_old).abs().max()
    sinv_old, sinv_new = torch.tensor(1 / s_old, device=DEV), torch.zeros((), device=DEV)
    got = cast.cast_to_fp8(xs, E4, sinv_old, scale_inv_out=sinv_new, amax_in=amax0, rescale=True)
    sinv_cpu = torch.zeros(())
    want = cast.cast_to_fp8(xs.cpu(), E4, sinv_old.cpu(), scale_inv_out=sinv_cpu, amax_in=amax0.cpu(), rescale=True)
    assert torch.equal(got.cpu(), want) and sinv_new.item() == sinv_cpu.item() and sinv_old.item() == 1 / s_old
    _status_ok()


@pytest.mark.parametrize('tile', [1, 2])
@pytest.mark.parametrize('layout', [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize('mnk', [(256, 256, 128), (512, 768, 1024), (1024, 512, 384), (400, 272, 200), (4096, 4096, 2048), (128, 16, 48)])
def test_gemm_layouts_and_tiles(mnk, layout, tile):
    """Every operand layout (K-major / MN-major) on the single-CTA and the CTA-pair kernel against fp32 math."""
    m, n, k = mnk
    a_mn, b_mn = layout
    if (a_mn != b_mn) and k % 16:
        k = (k + 15) // 16 * 16
    if (a_mn and m % 16) or (b_mn and n % 16):
        pytest.skip('the contiguous dimension must be a multiple of 16 bytes')
    a, sia = _mk(m, k, E5)
    b, sib = _mk(n, k, E4)
    ref = (a.view(F8[E5]).float() @ b.view(F8[E4]).float().t()) * (sia * sib)
    sc = ref.abs().max().item() + 1e-6
    aa = a.t().contiguous() if a_mn else a
    bb = b.t().contiguous() if b_mn else b
    d = gemm.gemm_fp8(aa, E5, sia, bb, E4, sib, torch.float32, a_mn=a_mn, b_mn=b_mn, tile=tile)
    assert (d - ref).abs().max().item() <= 1e-4 * sc + 1e-4
    _status_ok()


@pytest.mark.parametrize('tile', [1, 2])
def test_gemm_epilogue_options(tile):
    """Residual add, GeLU-derivative multiply, amax of the stored values, and the quantised copy of gelu(D)."""
    m, n, k = 512, 768, 512
    a, sia = _mk(m, k, E4)
    b, sib = _mk(n, k, E4)
    bias = torch.randn(n, device=DEV)
    ref = (a.view(F8[E4]).float() @ b.view(F8[E4]).float().t()) * (sia * sib)
    res = torch.randn(m, n, device=DEV).bfloat16()
    d = gemm.gemm_fp8(a, E4, sia, b, E4, sib, torch.bfloat16, bias=bias, residual=res, tile=tile)
    want = (ref + bias + res.float()).bfloat16()
    assert (d.float() - want.float()).abs().max().item() <= 0.02 * want.float().abs().max().item()
    # dgelu: product times gelu'(h)
    h = torch.randn(m, n, device=DEV).bfloat16()
    am = torch.zeros((), device=DEV)
    d = gemm.gemm_fp8(a, E4, sia, b, E4, sib, torch.bfloat16, gelu_src=h, amax_out=am, tile=tile)
    want = ref * gemm._gelu_tanh_grad(h.float())
    assert (d.float() - want).abs().max().item() <= 0.02 * want.abs().max().item()
    assert am.item() == d.float().abs().max().item()
    # forward of fc1: h = x W^T + b stored in bf16, amax and FP8 copy of gelu(h) from the same launch
    am = torch.zeros((), device=DEV)
    q_scale = torch.tensor(16.0, device=DEV)
    out8 = torch.empty(m, n, dtype=torch.uint8, device=DEV)
    d = gemm.gemm_fp8(a, E4, sia, b, E4, sib, torch.bfloat16, bias=bias, amax_out=am, act='gelu', out8=out8, out8_qtype=E4,
                      out8_scale=q_scale, tile=tile)
    g = K.gelu(d)    # the stand-alone kernel on the stored values
    assert am.item() == g.float().abs().max().item()
    assert torch.equal(out8, cast.cast_to_fp8(g, E4, q_scale))
    # backward of fc2 in the delayed regime: e5m2 copy of D = product x gelu'(h), its amax and its column sums (the bias
    # gradient of fc1) from one launch that does not store D itself; ragged and full tiles (513 rows, 768 / 800 columns)
    for mm, nn in ((m, n), (513, 800)):
        a2, sia2 = _mk(mm, k, E4)
        b2, sib2 = _mk(nn, k, E4)
        h2 = torch.randn(mm, nn, device=DEV).bfloat16()
        d_ref = gemm.gemm_fp8(a2, E4, sia2, b2, E4, sib2, torch.bfloat16, gelu_src=h2, tile=tile)
        am = torch.zeros((), device=DEV)
        cs = torch.full((nn, ), 7.0, device=DEV)
        q5 = torch.tensor(64.0, device=DEV)
        sinv = torch.zeros((), device=DEV)
        out5 = torch.empty(mm, nn, dtype=torch.uint8, device=DEV)
        none = gemm.gemm_fp8(a2, E4, sia2, b2, E4, sib2, torch.bfloat16, gelu_src=h2, amax_out=am, out8=out5, out8_qtype=E5, out8_scale=q5,
                             out8_scale_inv_out=sinv, colsum_out=cs, store_out=False, tile=tile)
        assert none is None
        assert am.item() == d_ref.float().abs().max().item() and sinv.item() == 1.0 / 64.0
        assert torch.equal(out5, cast.cast_to_fp8(d_ref, E5, q5))
        want_cs = d_ref.float().sum(0)
        assert (cs - want_cs).abs().max().item() <= 1e-3 * d_ref.float().abs().sum(0).max().item() + 1e-6
        # with D stored as well the same sums come out
        cs2 = torch.empty(nn, device=DEV)
        d2 = gemm.gemm_fp8(a2, E4, sia2, b2, E4, sib2, torch.bfloat16, gelu_src=h2, colsum_out=cs2, tile=tile)
        assert torch.equal(d2, d_ref)
        assert (cs2 - want_cs).abs().max().item() <= 1e-3 * d_ref.float().abs().sum(0).max().item() + 1e-6
    _status_ok()


def test_multi_tensor_norm_and_clip():
    """One launch for the norm over mixed high-precision / FP8 gradients, one for the clip, against torch on dequantised copies."""
    from msamp.ops import multi_tensor as mt
    torch.manual_seed(3)
    hp = [torch.randn(1000, 37, device=DEV), torch.randn(70001, device=DEV).bfloat16(), torch.randn(300, 300, device=DEV).half(),
          torch.randn(5, device=DEV)]
    fp8 = [(torch.randn(513, 129, device=DEV) * 0.01).cast(E4), (torch.randn(100000, device=DEV) * 3).cast(E5)]
    grads = hp + fp8
    want = sum(g.float().square().sum() for g in grads)
    stats = mt.grad_sumsq(grads, tag='test')
    assert stats[1].item() == 0 and abs(stats[0].item() - want.item()) <= 1e-4 * want.item()
    before = [g.float().clone() for g in grads]
    bytes_before = [g.value.clone() for g in fp8]
    max_norm = 0.25 * want.sqrt().item()
    mt.clip_by_sumsq(grads, stats[0:1], max_norm, tag='test')
    coef = max_norm / (want.sqrt().item() + 1e-6)
    for g, b in zip(grads, before):
        tol = 1e-2 if (not isinstance(g, torch.Tensor) or g.dtype != torch.float32) else 1e-6
        assert (g.float() - b * coef).abs().max().item() <= tol * (b.abs().max().item() * coef) + 1e-12
    assert all(torch.equal(g.value, b) for g, b in zip(fp8, bytes_before))    # FP8 gradients are clipped through scale_inv only
    # clipping with a generous threshold is a no-op; a non-finite value raises the flag
    again = [g.float().clone() for g in grads]
    mt.clip_by_sumsq(grads, mt.grad_sumsq(grads, tag='test')[0:1], 1e9, tag='test')
    assert all(torch.equal(g.float(), a) for g, a in zip(grads, again))
    hp[0][3, 3] = float('inf')
    assert mt.grad_sumsq(grads, tag='test')[1].item() == 1
    _status_ok()


def test_add_to_fp8_bit_exact():
    for q in (E4, E5):
        for dt in (torch.float32, torch.float16, torch.bfloat16):
            for n in (1, 63, 1024, 50001):
                x = torch.randn(n, device=DEV)
                t = x.cast(q)
                c = t.cpu()
                for _ in range(3):
                    other = torch.randn(n, device=DEV).to(dt)
                    arith.add_to_fp8(t.value, q, t.meta.scale, t.meta.scale_inv, t.meta.amax[0], other)
                    arith.add_to_fp8(c.value, q, c.meta.scale, c.meta.scale_inv, c.meta.amax[0], other.cpu())
                assert torch.equal(t.value.cpu(), c.value)
                assert t.meta.scale.item() == c.meta.scale.item() and t.meta.amax[0].item() == c.meta.amax[0].item()


def test_fp4_and_sumsq():
    x = (torch.randn(10007, device=DEV) * 3).bfloat16()
    assert torch.equal(arith.fp4_quantize_e2m1(x).cpu(), arith.fp4_quantize_e2m1(x.cpu()))
    d = arith.fp4_dge(x, 5.0, 3.0).float().cpu()
    r = arith.fp4_dge(x.cpu(), 5.0, 3.0).float()
    assert (d - r).abs().max().item() <= 0.02 * 3.0
    v = torch.randint(0, 0x78, (100003, ), dtype=torch.uint8, device=DEV)
    got = reduce.fp8_sumsq(v, E4).item()
    want = v.view(F8[E4]).float().square().sum().item()
    assert abs(got - want) <= 1e-4 * want


def _adam_case(p_kind, state_dtypes, use_adam, n):
    from msamp.optim import LBAdam, LBAdamW, LBAdamWBase
    torch.manual_seed(1)
    base = torch.randn(n)
    grads = [torch.randn(n) * 1e-2 for _ in range(4)]

    def make(dev):
        p = base.clone().to(dev)
        if p_kind == 'scaled16':
            from msamp.nn import ScalingParameter
            p = ScalingParameter(p.cast(Dtypes.kfloat16))
        else:
            p = p.to(p_kind).requires_grad_()
        return p

    pg, pc = make(DEV), make('cpu')
    kw = dict(lr=1e-2, weight_decay=1e-2, exp_avg_dtype=state_dtypes[0], exp_avg_sq_dtype=state_dtypes[1])
    og = (LBAdam if use_adam else LBAdamW)([pg], **kw)
    oc = LBAdamWBase([pc], **kw)
    oc.use_adam = use_adam
    for g in grads:
        if p_kind == 'scaled16':
            pg.grad, pc.grad = g.to(DEV).cast(E4), g.cast(E4)
        else:
            pg.grad, pc.grad = g.to(DEV).to(p_kind), g.to(p_kind)
        og.step()
        oc.step()
    fg = pg.float().cpu()
    fc = pc.float()
    return fg, fc, og.state[pg], oc.state[pc]


@pytest.mark.parametrize('p_kind', ['scaled16', torch.float32, torch.bfloat16])
@pytest.mark.parametrize('state_dtypes', [(torch.uint8, torch.float16), (torch.float32, torch.float32), (torch.int8, torch.float16)])
@pytest.mark.parametrize('use_adam', [False, True])
def test_fused_adam_matches_definition(p_kind, state_dtypes, use_adam):
    for n in (5, 4096 + 3, 70001):
        fg, fc, sg, sc = _adam_case(p_kind, state_dtypes, use_adam, n)
        tol = 5e-2 if p_kind == torch.bfloat16 else (1e-2 if p_kind == 'scaled16' else 2e-3)    # a few ulps of the storage format
        if state_dtypes[0] == torch.int8:
            tol *= 3    # e5m2 moments carry two mantissa bits
        assert (fg - fc).abs().max().item() <= tol, (fg - fc).abs().max()
        mg, mc = sg['exp_avg'].float().cpu(), sc['exp_avg'].float()
        vg, vc = sg['exp_avg_sq'].float().cpu(), sc['exp_avg_sq'].float()
        assert (mg - mc).abs().max().item() <= (0.26 if state_dtypes[0] == torch.int8 else 0.13) * mc.abs().max().item() + 1e-7    # one fp8 step at the top of the range
        assert (vg - vc).abs().max().item() <= 0.02 * vc.abs().max().item() + 1e-9


@pytest.mark.parametrize('dt', [torch.bfloat16, torch.float32])
@pytest.mark.parametrize('shape', [(64, 256), (1000, 4096), (7, 1024), (3, 8192), (2500, 4096), (1300, 1024)])    # the last two: bulk-copy backward
def test_layernorm(dt, shape):
    if dt == torch.float32 and shape[1] > 4096:
        pytest.skip('rows of fp32 data are limited to 4096 columns')
    torch.manual_seed(0)
    x = (torch.randn(*shape, device=DEV) * 2 + 0.5).to(dt).requires_grad_()
    w = (torch.rand(shape[1], device=DEV) + 0.5).requires_grad_()
    b = torch.randn(shape[1], device=DEV).requires_grad_()
    y = K.layer_norm(x, w, b, 1e-5)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    wr, br = w.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    yr = torch.nn.functional.layer_norm(xr, (shape[1], ), wr, br, 1e-5)
    yr.backward(dy.float())
    tol = 3e-2 if dt == torch.bfloat16 else 1e-4
    assert (y.float() - yr).abs().max().item() <= tol
    assert (x.grad.float() - xr.grad).abs().max().item() <= tol * 2
    assert (w.grad - wr.grad).abs().max().item() <= tol * math.sqrt(shape[0]) * 2
    assert (b.grad - br.grad).abs().max().item() <= tol * math.sqrt(shape[0]) * 2


@pytest.mark.parametrize('shape', [(64, 1024), (300, 4096), (17, 8192), (2500, 4096), (1500, 2048)])
def test_layernorm_quantised_output_and_residual_backward(shape):
    """LayerNorm that emits e4m3 directly == LayerNorm followed by the cast, bit for bit; backward with the skip gradient."""
    torch.manual_seed(0)
    x = (torch.randn(*shape, device=DEV) * 2 + 0.5).bfloat16()
    w = torch.rand(shape[1], device=DEV) + 0.5
    b = torch.randn(shape[1], device=DEV)
    y, _, mean, rstd = K.layer_norm_fwd_raw(x, w, b, 1e-5)
    # delayed regime: given scale, amax recorded
    scale, am, si = torch.tensor(16.0, device=DEV), torch.zeros((), device=DEV), torch.zeros((), device=DEV)
    _, y8, mean2, rstd2 = K.layer_norm_fwd_raw(x, w, b, 1e-5, want_y=False, want_y8=True, y8_scale=scale, amax_out=am, scale_inv_out=si)
    assert torch.equal(y8, cast.cast_to_fp8(y, E4, scale)) and am.item() == y.float().abs().max().item() and si.item() == 1 / 16
    assert torch.equal(mean, mean2) and torch.equal(rstd, rstd2)
    # in-time regime: statistics pass, then the scale follows from the amax
    am2 = torch.zeros((), device=DEV)
    K.layer_norm_fwd_raw(x, w, b, 1e-5, want_y=False, amax_out=am2)
    assert am2.item() == am.item()
    scale2, si2 = torch.ones((), device=DEV), torch.zeros((), device=DEV)
    _, y8b, _, _ = K.layer_norm_fwd_raw(x, w, b, 1e-5, want_y=False, want_y8=True, y8_scale=scale2, amax_in=am2, scale_inv_out=si2)
    want_scale = cast.compute_scale(am2, torch.ones((), device=DEV), 448.0)
    assert scale2.item() == want_scale.item() and si2.item() == 1 / want_scale.item()
    assert torch.equal(y8b, cast.cast_to_fp8(y, E4, want_scale))
    # backward: dx = LayerNorm'(dy) + dres, with max|dx|
    dy, dres = torch.randn_like(y), torch.randn_like(y)
    dx0, dg0, db0 = K.layer_norm_bwd_raw(dy, x, w, mean, rstd, True)
    amx = torch.zeros((), device=DEV)
    dx1, dg1, db1 = K.layer_norm_bwd_raw(dy, x, w, mean, rstd, True, dres=dres, amax_out=amx)
    ref = K.layer_norm_bwd_raw(dy.cpu(), x.cpu(), w.cpu(), mean.cpu(), rstd.cpu(), True, dres=dres.cpu())[0]
    assert (dx1.float().cpu() - ref.float()).abs().max().item() <= 4e-2
    assert (dx1.float() - (dx0.float() + dres.float())).abs().max().item() <= 4e-2
    assert amx.item() == dx1.float().abs().max().item()
    assert torch.equal(dg0, dg1) and torch.equal(db0, db1)
    _status_ok()


def test_gelu():
    x = torch.randn(100003, device=DEV, dtype=torch.bfloat16).requires_grad_()
    y = K.gelu(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = torch.nn.functional.gelu(xr, approximate='tanh')
    yr.backward(dy.float())
    assert (y.float() - yr).abs().max().item() <= 2e-2
    assert (x.grad.float() - xr.grad).abs().max().item() <= 3e-2


def _attn_ref(q, k, v, causal):
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    s = (qf @ kf.transpose(-1, -2)) / math.sqrt(q.shape[-1])
    if causal:
        S = q.shape[1]
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device=q.device).triu(1), float('-inf'))
    return (torch.softmax(s, -1) @ vf).permute(0, 2, 1, 3)


@pytest.mark.parametrize('d', [64, 128])
@pytest.mark.parametrize('S', [64, 128, 200, 512])
@pytest.mark.parametrize('causal', [True, False])
def test_attention(d, S, causal):
    torch.manual_seed(0)
    B, H = 2, 3
    qkv = torch.randn(B, S, 3, H, d, device=DEV, dtype=torch.bfloat16).requires_grad_()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    o = K.attention(q, k, v, causal=causal, grad_layout='packed')
    do = torch.randn_like(o)
    o.backward(do)
    ref_in = qkv.detach().float().requires_grad_()
    r = _attn_ref(ref_in[:, :, 0], ref_in[:, :, 1], ref_in[:, :, 2], causal)
    r.backward(do.float())
    assert (o.float() - r).abs().max().item() <= 3e-2
    err = (qkv.grad.float() - ref_in.grad).abs().max().item()
    assert err <= 6e-2 * max(1.0, ref_in.grad.abs().max().item()), err
    # the packed entry point gives the same numbers
    qkv3 = qkv.detach().clone().requires_grad_()
    o3 = K.attention_qkv(qkv3, causal=causal)
    o3.backward(do)
    assert torch.equal(o3, o) and torch.equal(qkv3.grad, qkv.grad)
    # separate tensors / separate gradients
    q2, k2, v2 = (t.detach().contiguous().requires_grad_() for t in (q, k, v))
    o2 = K.attention(q2, k2, v2, causal=causal)
    o2.backward(do)
    assert torch.equal(o2, o)
    assert (q2.grad.float() - ref_in.grad[:, :, 0]).abs().max().item() <= 6e-2 * max(1.0, ref_in.grad.abs().max().item())


@pytest.mark.parametrize('impl', ['tc', 'mma'])
def test_attention_long_rows_growing_maximum(impl, monkeypatch):
    """Head size 128 through both kernel families; the scores grow along the key axis so that the
    running maximum keeps rising (the tcgen05 forward rescales its TMEM accumulator on the way)."""
    monkeypatch.setenv('MSAMP_ATTN_IMPL', impl)
    torch.manual_seed(1)
    B, S, H, d = 1, 1280, 2, 128
    qkv = torch.randn(B, S, 3, H, d, device=DEV)
    qkv[:, :, 1] *= torch.linspace(0.2, 6.0, S, device=DEV).view(1, S, 1, 1)    # later keys score higher
    qkv = qkv.bfloat16().requires_grad_()
    o = K.attention_qkv(qkv, causal=True)
    do = torch.randn_like(o)
    o.backward(do)
    assert native.device_status() == 0
    ref_in = qkv.detach().float().requires_grad_()
    r = _attn_ref(ref_in[:, :, 0], ref_in[:, :, 1], ref_in[:, :, 2], True)
    r.backward(do.float())
    assert (o.float() - r).abs().max().item() <= 4e-2
    for i in range(3):
        g, gr = qkv.grad[:, :, i].float(), ref_in.grad[:, :, i]
        assert (g - gr).abs().max().item() <= 3e-2 * max(1.0, gr.abs().max().item())


@pytest.mark.parametrize('causal', [True, False])
def test_attention_more_work_items_than_sms(causal):
    """The tcgen05 kernels are persistent: with more (tile, batch, head) items than SMs every CTA walks several items
    (rings, score slots and barriers keep running across them; the last wave is partial).  3 x 8 heads x 1536 = 288 items."""
    torch.manual_seed(2)
    B, S, H, d = 3, 1536, 8, 128
    qkv = torch.randn(B, S, 3, H, d, device=DEV).bfloat16().requires_grad_()
    o = K.attention_qkv(qkv, causal=causal)
    do = torch.randn_like(o)
    o.backward(do)
    assert native.device_status() == 0
    ref_in = qkv.detach().float().requires_grad_()
    r = _attn_ref(ref_in[:, :, 0], ref_in[:, :, 1], ref_in[:, :, 2], causal)
    r.backward(do.float())
    assert (o.float() - r).abs().max().item() <= 3e-2
    for i in range(3):
        g, gr = qkv.grad[:, :, i].float(), ref_in.grad[:, :, i]
        assert (g - gr).abs().max().item() <= 3e-2 * max(1.0, gr.abs().max().item()), i
    # a second call gives the same bits (the kernels are deterministic and leave no state behind)
    qkv2 = qkv.detach().clone().requires_grad_()
    o2 = K.attention_qkv(qkv2, causal=causal)
    o2.backward(do)
    assert torch.equal(o2, o) and torch.equal(qkv2.grad, qkv.grad)


_ATTN_VARIANT_SCRIPT = """
import math, sys, torch
sys.path.insert(0, %r)
from msamp.ops import native, nn as K
torch.manual_seed(3)
B, S, H, d = 2, 640, 4, 128
qkv = torch.randn(B, S, 3, H, d, device='cuda').bfloat16().requires_grad_()
o = K.attention_qkv(qkv, causal=True)
do = torch.randn_like(o)
o.backward(do)
assert native.device_status() == 0
ref = qkv.detach().float().requires_grad_()
q, k, v = (ref[:, :, i].permute(0, 2, 1, 3) for i in range(3))
s = (q @ k.transpose(-1, -2)) / math.sqrt(d)
s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device='cuda').triu(1), float('-inf'))
r = (torch.softmax(s, -1) @ v).permute(0, 2, 1, 3)
r.backward(do.float())
assert (o.float() - r).abs().max().item() <= 3e-2
assert (qkv.grad.float() - ref.grad).abs().max().item() <= 3e-2 * max(1.0, ref.grad.abs().max().item())
print('ok')
"""


@pytest.mark.parametrize('env', [{'MSAMP_ATTN_FWD_PERSIST': '0', 'MSAMP_ATTN_BWD_PERSIST': '0'},
                                 {'MSAMP_ATTN_FWD_SMEM': '1', 'MSAMP_ATTN_BWD_SMEM': '1'}])
def test_attention_kernel_variants(env):
    """The earlier attention kernels stay selectable through environment variables that are read once per process
    (one CTA per work item instead of persistent CTAs; 64-wide score tiles with P / dS in shared memory): each
    combination runs in a fresh process against the fp32 reference."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, '-c', _ATTN_VARIANT_SCRIPT % root], env=dict(os.environ, **env), capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0 and 'ok' in res.stdout, res.stderr[-2000:]


def test_cross_entropy():
    torch.manual_seed(0)
    rows, vocab = 300, 50304
    logits = (torch.randn(rows, vocab, device=DEV) * 2).bfloat16().requires_grad_()
    target = torch.randint(0, vocab, (rows, ), device=DEV)
    target[3] = -100
    ref_l = logits.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(ref_l, target, ignore_index=-100)
    ref.backward()
    work = logits.detach().clone().requires_grad_()
    loss = K.cross_entropy(work, target)
    loss.backward()
    assert abs(loss.item() - ref.item()) <= 1e-3
    assert (work.grad.float() - ref_l.grad).abs().max().item() <= 1e-4
