"""Fused transformer sublayers on FP8 linears: LayerNorm→Linear, LayerNorm→QKV→attention→proj(+skip) and
LayerNorm→fc1→GeLU→fc2(+skip), each as ONE autograd function.

What the fusion buys over composing ``layer_norm``, ``F.linear``, ``gelu`` and ``+`` (the sequence of the reference's
FP8 linear, msamp/nn/functional.py:19-125, around TE-style LayerNorm / GeLU kernels):

* an activation that only feeds an FP8 GEMM is never written in 16 bits: LayerNorm emits e4m3 directly, GeLU is
  folded into the quantising pass (or, once the amax history drives the scale, into the fc1 GEMM epilogue);
* the skip connection is added in the epilogue of the proj / fc2 GEMM, its gradient inside the LayerNorm-backward
  kernel; the GeLU derivative is applied in the epilogue of the fc2 dgrad GEMM;
* in the in-time scaling regime (window 1 or warm-up) the amax a cast needs comes from the kernel that produced
  the tensor (GEMM epilogue, LayerNorm forward / backward) instead of an extra pass;
* every FP8 operand is quantised once and read in its own layout by forward, dgrad and wgrad.

The quantisation semantics (formats, metas ``input`` / ``wgrad`` / ``ograd`` of each FP8Linear, window sizes, weight
gradients delivered through ``weight.backward_grad_update``) are those of ``msamp.nn.functional._FP8GemmFunction``;
the code runs on CPU tensors through the same bit-exact emulation of each operator.
"""
import torch

from msamp.common.dtype import Dtypes
from msamp.nn.functional import _quantize_wgrad, gemm_dgrad, gemm_wgrad, weight_fp8
from msamp.nn.parameter import ScalingParameter
from msamp.nn.state import model_state
from msamp.ops import cast as _k
from msamp.ops import gemm as _g
from msamp.ops import nn as _nn

E4M3, E5M2 = Dtypes.kfloat8_e4m3, Dtypes.kfloat8_e5m2
_AMAX_HINT = '_msamp_amax'    # attribute by which a producer hands max|t| of a tensor it wrote to the next quantiser


def fusable(*linears):
    """True if every module is an FP8Linear whose weight is a ScalingParameter (not an FSDP flat view)."""
    return all(isinstance(getattr(m, 'weight', None), ScalingParameter) and hasattr(m, 'scaling_metas') for m in linears)


def _quantize(x, meta, qtype, act=None, colsum=None, amax_hint=None):
    """``x`` → FP8 bytes under ``meta`` (in-time or delayed scaling); returns ``(bytes, scale_inv snapshot)``.

    ``amax_hint`` is a 0-d tensor that already holds ``max|act(x)|``; it is only used (and only needed) in the in-time regime.
    """
    if meta.is_in_time_scaling():
        if amax_hint is None:
            if act is not None:
                raise RuntimeError('an activation folded into the cast needs the amax of its result')
            _k.amax_and_scale(x, meta.amax[0], meta.scale, meta.scale_inv, qtype)
            x8 = _k.cast_to_fp8(x, qtype, meta.scale, colsum_out=colsum)
        elif amax_hint.data_ptr() == meta.amax[0].data_ptr():
            x8 = _k.cast_to_fp8(x, qtype, meta.scale, scale_inv_out=meta.scale_inv, amax_in=amax_hint, act=act, colsum_out=colsum)
        else:
            # the cast re-records the amax (same value) into the meta while it derives the scale from the hint
            x8 = _k.cast_to_fp8(x, qtype, meta.scale, meta.amax[0], scale_inv_out=meta.scale_inv, amax_in=amax_hint, act=act,
                                colsum_out=colsum)
    else:
        x8 = _k.cast_to_fp8(x, qtype, meta.scale, meta.amax[0], scale_inv_out=meta.scale_inv, act=act, colsum_out=colsum)
    return x8, meta.scale_inv.clone()


def _ln_quantize(x, ln_weight, ln_bias, eps, meta):
    """LayerNorm whose output exists only as e4m3 bytes; returns ``(y8, scale_inv snapshot, mean, rstd)``."""
    if meta.is_in_time_scaling():
        # pass 1: row statistics and max|y|; pass 2: normalise again and quantise with the scale that amax implies
        _nn.layer_norm_fwd_raw(x, ln_weight, ln_bias, eps, want_y=False, amax_out=meta.amax[0])
        _, y8, mean, rstd = _nn.layer_norm_fwd_raw(x, ln_weight, ln_bias, eps, want_y=False, want_y8=True, y8_scale=meta.scale,
                                                   amax_in=meta.amax[0], scale_inv_out=meta.scale_inv)
    else:
        _, y8, mean, rstd = _nn.layer_norm_fwd_raw(x, ln_weight, ln_bias, eps, want_y=False, want_y8=True, y8_scale=meta.scale,
                                                   amax_out=meta.amax[0], scale_inv_out=meta.scale_inv)
    return y8, meta.scale_inv.clone(), mean, rstd


def _deliver_wgrad(weight, metas, dy8, dy_sinv, x8, x_sinv, out_dtype):
    """Weight gradient ``dy8ᵀ · x8`` → quantised ScalingTensor handed to the parameter (accumulating in high precision)."""
    if not weight.requires_grad:
        return
    wg_meta = metas['wgrad']
    amax0 = wg_meta.amax[0]
    if weight.grad is None:
        wgrad = gemm_wgrad(dy8, dy_sinv, x8, x_sinv, out_dtype, amax_out=amax0)
    else:
        old = weight.grad.to(out_dtype)
        wgrad = gemm_wgrad(dy8, dy_sinv, x8, x_sinv, out_dtype, accumulate=True, out=old, amax_out=amax0)
    wgrad = wgrad.view(weight.shape)
    if model_state.use_fp8_ddp:
        wgrad.meta = wg_meta    # the FP8 DDP reducer quantises whole buckets with a cross-rank scale
    else:
        wgrad = _quantize_wgrad(wgrad, wg_meta, out=getattr(weight, '_grad_out', None))
    weight.backward_grad_update(wgrad)


def _quantize_ograd(dy, meta, has_bias, bias_dtype):
    """Output gradient → e5m2 bytes; the bias gradient (column sums) comes out of the same pass."""
    colsum = torch.zeros(dy.shape[1], dtype=torch.float32, device=dy.device) if has_bias else None
    dy8, dy_sinv = _quantize(dy, meta, E5M2, colsum=colsum, amax_hint=getattr(dy, _AMAX_HINT, None))
    return dy8, dy_sinv, (colsum.to(bias_dtype) if has_bias else None)


def _ln_backward(dln, x, ln_weight, mean, rstd, has_ln_bias, dres):
    """LayerNorm backward + skip-connection gradient; tags the result with its amax for the next quantiser."""
    amax = torch.empty((), dtype=torch.float32, device=x.device)
    dx, dgamma, dbeta = _nn.layer_norm_bwd_raw(dln, x, ln_weight, mean, rstd, has_ln_bias, dres=dres, amax_out=amax)
    setattr(dx, _AMAX_HINT, amax)
    return dx, dgamma, dbeta


class _LnLinearFn(torch.autograd.Function):
    """``linear(layer_norm(x))`` (the reference composes TE's LayerNorm with msamp/nn/functional.py:19-125)."""
    @staticmethod
    def forward(ctx, x, ln_weight, ln_bias, bias, eps, weight, metas):
        model_state.check_metas_in_flat(metas)
        x = x.contiguous()
        y8, y_sinv, mean, rstd = _ln_quantize(x, ln_weight, ln_bias, eps, metas['input'])
        w8, w_sinv = weight_fp8(weight)
        out = _g.gemm_fp8(y8, E4M3, y_sinv, w8, E4M3, w_sinv, x.dtype, bias=bias)
        ctx.save_for_backward(x, ln_weight, mean, rstd, y8, y_sinv, w8, w_sinv)
        ctx.weight, ctx.metas = weight, metas
        ctx.has_ln_bias, ctx.bias_dtype = ln_bias is not None, (bias.dtype if bias is not None else None)
        return out

    @staticmethod
    def backward(ctx, dy):
        x, ln_weight, mean, rstd, y8, y_sinv, w8, w_sinv = ctx.saved_tensors
        metas = ctx.metas
        dy = dy.contiguous()
        dy8, dy_sinv, dbias = _quantize_ograd(dy, metas['ograd'], ctx.bias_dtype is not None, ctx.bias_dtype)
        _deliver_wgrad(ctx.weight, metas, dy8, dy_sinv, y8, y_sinv, x.dtype)
        dln = gemm_dgrad(dy8, dy_sinv, w8, w_sinv, x.dtype)
        dx, dgamma, dbeta = _ln_backward(dln, x, ln_weight, mean, rstd, ctx.has_ln_bias, None)
        return dx, dgamma, dbeta, dbias, None, None, None


class _MlpSublayerFn(torch.autograd.Function):
    """``x + fc2(gelu(fc1(layer_norm(x))))`` (without the ``x +`` when ``add_residual`` is false)."""
    @staticmethod
    def forward(ctx, x, ln_weight, ln_bias, b1, b2, eps, w1, m1, w2, m2, add_residual=True):
        model_state.check_metas_in_flat(m1)
        model_state.check_metas_in_flat(m2)
        x = x.contiguous()
        dt = x.dtype
        y8, y_sinv, mean, rstd = _ln_quantize(x, ln_weight, ln_bias, eps, m1['input'])
        w1_8, w1_sinv = weight_fp8(w1)
        w2_8, w2_sinv = weight_fp8(w2)
        g_meta = m2['input']
        if g_meta.is_in_time_scaling():
            # fc1 epilogue reduces max|gelu(h)|; the quantising pass applies GeLU and the scale that amax implies
            h = _g.gemm_fp8(y8, E4M3, y_sinv, w1_8, E4M3, w1_sinv, dt, bias=b1, amax_out=g_meta.amax[0], act='gelu')
            g8, g_sinv = _quantize(h, g_meta, E4M3, act='gelu', amax_hint=g_meta.amax[0])
        else:
            # the scale is known: the fc1 epilogue writes gelu(h) as e4m3 next to h and records its amax
            g8 = torch.empty((x.shape[0], w1_8.shape[0]), dtype=torch.uint8, device=x.device)
            h = _g.gemm_fp8(y8, E4M3, y_sinv, w1_8, E4M3, w1_sinv, dt, bias=b1, amax_out=g_meta.amax[0], act='gelu', out8=g8,
                            out8_qtype=E4M3, out8_scale=g_meta.scale, out8_scale_inv_out=g_meta.scale_inv)
            g_sinv = g_meta.scale_inv.clone()
        out = _g.gemm_fp8(g8, E4M3, g_sinv, w2_8, E4M3, w2_sinv, dt, bias=b2, residual=x if add_residual else None)
        ctx.add_residual = add_residual
        ctx.save_for_backward(x, ln_weight, mean, rstd, y8, y_sinv, h, g8, g_sinv, w1_8, w1_sinv, w2_8, w2_sinv)
        ctx.w1, ctx.m1, ctx.w2, ctx.m2 = w1, m1, w2, m2
        ctx.has_ln_bias = ln_bias is not None
        ctx.b1_dtype = b1.dtype if b1 is not None else None
        ctx.b2_dtype = b2.dtype if b2 is not None else None
        return out

    @staticmethod
    def backward(ctx, g):
        x, ln_weight, mean, rstd, y8, y_sinv, h, g8, g_sinv, w1_8, w1_sinv, w2_8, w2_sinv = ctx.saved_tensors
        m1, m2 = ctx.m1, ctx.m2
        dt = x.dtype
        g = g.contiguous()
        # fc2
        dy8, dy_sinv, db2 = _quantize_ograd(g, m2['ograd'], ctx.b2_dtype is not None, ctx.b2_dtype)
        _deliver_wgrad(ctx.w2, m2, dy8, dy_sinv, g8, g_sinv, dt)
        # dgrad of fc2 with the GeLU derivative applied in the epilogue
        og = m1['ograd']
        if og.is_in_time_scaling():
            # in-time scaling: the scale of dh follows from its amax, which the epilogue reduces on the way; the
            # quantisation (and the bias gradient) is a second pass over dh
            dh_amax = torch.empty((), dtype=torch.float32, device=x.device)
            dh = gemm_dgrad(dy8, dy_sinv, w2_8, w2_sinv, dt, gelu_src=h, amax_out=dh_amax)
            setattr(dh, _AMAX_HINT, dh_amax)
            dh8, dh_sinv, db1 = _quantize_ograd(dh, og, ctx.b1_dtype is not None, ctx.b1_dtype)
            del dh
        else:
            # delayed scaling: the scale is known beforehand, so the epilogue writes the e5m2 operand of the next two GEMMs,
            # the amax for the history and the column sums (= the bias gradient of fc1) itself; dh in bf16 is never stored
            dh8 = torch.empty((dy8.shape[0], h.shape[1]), dtype=torch.uint8, device=x.device)
            colsum = torch.empty(h.shape[1], dtype=torch.float32, device=x.device) if ctx.b1_dtype is not None else None
            gemm_dgrad(dy8, dy_sinv, w2_8, w2_sinv, dt, gelu_src=h, amax_out=og.amax[0], out8=dh8, out8_qtype=E5M2, out8_scale=og.scale,
                       out8_scale_inv_out=og.scale_inv, colsum_out=colsum, store_out=False)
            dh_sinv = og.scale_inv.clone()
            db1 = colsum.to(ctx.b1_dtype) if colsum is not None else None
        # fc1
        _deliver_wgrad(ctx.w1, m1, dh8, dh_sinv, y8, y_sinv, dt)
        dln = gemm_dgrad(dh8, dh_sinv, w1_8, w1_sinv, dt)
        dx, dgamma, dbeta = _ln_backward(dln, x, ln_weight, mean, rstd, ctx.has_ln_bias, g if ctx.add_residual else None)
        return dx, dgamma, dbeta, db1, db2, None, None, None, None, None, None


class _AttnSublayerFn(torch.autograd.Function):
    """``x + proj(attention(qkv(layer_norm(x))))`` with causal softmax attention on the packed QKV projection."""
    @staticmethod
    def forward(ctx, x, ln_weight, ln_bias, b_qkv, b_proj, eps, w_qkv, m_qkv, w_proj, m_proj, batch, seq, n_head, causal):
        model_state.check_metas_in_flat(m_qkv)
        model_state.check_metas_in_flat(m_proj)
        x = x.contiguous()
        dt = x.dtype
        y8, y_sinv, mean, rstd = _ln_quantize(x, ln_weight, ln_bias, eps, m_qkv['input'])
        wq8, wq_sinv = weight_fp8(w_qkv)
        wp8, wp_sinv = weight_fp8(w_proj)
        qkv = _g.gemm_fp8(y8, E4M3, y_sinv, wq8, E4M3, wq_sinv, dt, bias=b_qkv)
        head_dim = qkv.shape[1] // (3 * n_head)
        qkv5 = qkv.view(batch, seq, 3, n_head, head_dim)
        o, lse = _nn.attention_qkv_fwd_raw(qkv5, causal)
        o2 = o.view(batch * seq, n_head * head_dim)
        o8, o_sinv = _quantize(o2, m_proj['input'], E4M3)
        out = _g.gemm_fp8(o8, E4M3, o_sinv, wp8, E4M3, wp_sinv, dt, bias=b_proj, residual=x)
        ctx.save_for_backward(x, ln_weight, mean, rstd, y8, y_sinv, qkv, o, lse, o8, o_sinv, wq8, wq_sinv, wp8, wp_sinv)
        ctx.w_qkv, ctx.m_qkv, ctx.w_proj, ctx.m_proj = w_qkv, m_qkv, w_proj, m_proj
        ctx.shape = (batch, seq, n_head, head_dim)
        ctx.causal = causal
        ctx.has_ln_bias = ln_bias is not None
        ctx.bq_dtype = b_qkv.dtype if b_qkv is not None else None
        ctx.bp_dtype = b_proj.dtype if b_proj is not None else None
        return out

    @staticmethod
    def backward(ctx, g):
        x, ln_weight, mean, rstd, y8, y_sinv, qkv, o, lse, o8, o_sinv, wq8, wq_sinv, wp8, wp_sinv = ctx.saved_tensors
        m_qkv, m_proj = ctx.m_qkv, ctx.m_proj
        batch, seq, n_head, head_dim = ctx.shape
        dt = x.dtype
        g = g.contiguous()
        # proj
        dy8, dy_sinv, dbp = _quantize_ograd(g, m_proj['ograd'], ctx.bp_dtype is not None, ctx.bp_dtype)
        _deliver_wgrad(ctx.w_proj, m_proj, dy8, dy_sinv, o8, o_sinv, dt)
        d_o = gemm_dgrad(dy8, dy_sinv, wp8, wp_sinv, dt)
        # attention
        dqkv = _nn.attention_qkv_bwd_raw(qkv.view(batch, seq, 3, n_head, head_dim), o, lse, d_o.view(batch, seq, n_head, head_dim), ctx.causal)
        del d_o
        dqkv2 = dqkv.view(batch * seq, 3 * n_head * head_dim)
        # qkv
        dq8, dq_sinv, dbq = _quantize_ograd(dqkv2, m_qkv['ograd'], ctx.bq_dtype is not None, ctx.bq_dtype)
        del dqkv, dqkv2
        _deliver_wgrad(ctx.w_qkv, m_qkv, dq8, dq_sinv, y8, y_sinv, dt)
        dln = gemm_dgrad(dq8, dq_sinv, wq8, wq_sinv, dt)
        dx, dgamma, dbeta = _ln_backward(dln, x, ln_weight, mean, rstd, ctx.has_ln_bias, g)
        return dx, dgamma, dbeta, dbq, dbp, None, None, None, None, None, None, None, None, None


def ln_linear(x, ln, linear):
    """``linear(ln(x))`` for a LayerNorm-like module (``weight``, ``bias``, ``eps``) and an FP8Linear, 2-D ``x``."""
    model_state.ready_to_scale_tensor = True    # the optimizer rolls the amax windows only after an FP8 forward ran
    return _LnLinearFn.apply(x, ln.weight, ln.bias, linear.bias, ln.eps, linear.weight, linear.scaling_metas)


def mlp_sublayer(x, ln, fc1, fc2, residual=True):
    """``x + fc2(gelu(fc1(ln(x))))`` for FP8Linear ``fc1`` / ``fc2``, 2-D ``x``; ``residual=False`` drops the ``x +``."""
    model_state.ready_to_scale_tensor = True
    return _MlpSublayerFn.apply(x, ln.weight, ln.bias, fc1.bias, fc2.bias, ln.eps, fc1.weight, fc1.scaling_metas, fc2.weight,
                                fc2.scaling_metas, bool(residual))


class ModuleView:
    """Presents parameters that live under other names (e.g. ``layer_norm_weight``, ``fc1_weight`` of the TE-shaped
    modules) as the ``weight`` / ``bias`` / ``eps`` / ``scaling_metas`` attributes the sublayer functions read."""
    def __init__(self, weight, bias=None, eps=None, scaling_metas=None):
        self.weight, self.bias, self.eps, self.scaling_metas = weight, bias, eps, scaling_metas


def attention_sublayer(x, ln, qkv, proj, batch, seq, n_head, causal=True):
    """``x + proj(attention(qkv(ln(x))))`` for FP8Linear ``qkv`` (packed ``[3 * hidden, hidden]``) and ``proj``, 2-D ``x``."""
    model_state.ready_to_scale_tensor = True
    return _AttnSublayerFn.apply(x, ln.weight, ln.bias, qkv.bias, proj.bias, ln.eps, qkv.weight, qkv.scaling_metas, proj.weight,
                                 proj.scaling_metas, batch, seq, n_head, causal)
