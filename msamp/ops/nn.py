"""Transformer-block operators (LayerNorm, GeLU, attention, cross-entropy) as autograd functions.

CUDA tensors use the kernels in ``csrc/nn.cu`` and ``csrc/attention.cu``; CPU tensors use plain
torch math (the oracle the GPU tests compare against).
"""
import ctypes
import math
import os

import torch
import torch.nn.functional as F

from msamp.ops import native

_i64x24 = ctypes.c_int64 * 24


def _use_native(t):
    return t.is_cuda


# ---------------------------------------------------------------------------------------- LayerNorm
class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        rows, cols = x2.shape
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        native.check(
            native.lib().msamp_layernorm_fwd(
                native.ptr(x2), native.ptr(weight), native.ptr(bias), native.dt(x2.dtype), native.dt(weight.dtype), native.ptr(y),
                native.ptr(mean), native.ptr(rstd), rows, cols, ctypes.c_float(eps), native.stream()
            ), 'layernorm_fwd'
        )
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.has_bias = bias is not None
        ctx.shape = shape
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, mean, rstd = ctx.saved_tensors
        rows, cols = x2.shape
        dy2 = dy.reshape(rows, cols).contiguous()
        dx = torch.empty_like(x2)
        dgamma = torch.empty_like(weight)
        dbeta = torch.empty_like(weight) if ctx.has_bias else None
        nparts = native.lib().msamp_layernorm_bwd_parts()
        part = torch.empty(nparts * 2 * cols, dtype=torch.float32, device=x2.device)
        native.check(
            native.lib().msamp_layernorm_bwd(
                native.ptr(dy2), native.ptr(x2), native.ptr(weight), native.dt(x2.dtype), native.dt(weight.dtype), native.ptr(mean),
                native.ptr(rstd), native.ptr(dx), native.ptr(dgamma), native.ptr(dbeta), native.ptr(part), rows, cols, native.stream()
            ), 'layernorm_bwd'
        )
        return dx.view(ctx.shape), dgamma, dbeta, None


def _ln_supported(x, weight, bias):
    cols = x.shape[-1]
    vec = 4 if x.dtype == torch.float32 else 8
    return (cols % vec == 0 and cols <= native.lib().msamp_layernorm_max_cols(native.dt(x.dtype))
            and weight.dtype in (torch.float32, torch.float16, torch.bfloat16) and (bias is None or bias.dtype == weight.dtype))


def layer_norm_fwd_raw(x2, weight, bias, eps, want_y=True, y8_scale=None, amax_in=None, amax_out=None, scale_inv_out=None, want_y8=False):
    """LayerNorm forward without autograd on a contiguous 2-D ``x2``.

    Returns ``(y or None, y8 or None, mean, rstd)``.  ``y8`` is the e4m3 copy of the output quantised with
    ``y8_scale`` (a 0-d fp32 tensor); with ``amax_in`` the scale is first derived from that amax by the power-of-two
    rule and written back to ``y8_scale``.  ``amax_out`` receives ``max|y|`` and ``scale_inv_out`` ``1 / scale``.
    The quantised values are taken from the output as rounded to the dtype of ``x2``, so they equal a separate cast
    of ``y`` bit for bit.  With ``want_y=False`` and ``want_y8=False`` only the statistics and ``amax_out`` are produced.
    """
    rows, cols = x2.shape
    if x2.is_cuda:
        if not _ln_supported(x2, weight, bias):
            raise RuntimeError(f'layer_norm: unsupported shape/dtype on CUDA (cols={cols}, dtype={x2.dtype}, param={weight.dtype})')
        y = torch.empty_like(x2) if want_y else None
        y8 = torch.empty((rows, cols), dtype=torch.uint8, device=x2.device) if want_y8 else None
        mean = torch.empty(rows, dtype=torch.float32, device=x2.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x2.device)
        native.check(
            native.lib().msamp_layernorm_fwd_q(
                native.ptr(x2), native.ptr(weight), native.ptr(bias), native.dt(x2.dtype), native.dt(weight.dtype), native.ptr(y),
                native.ptr(mean), native.ptr(rstd), rows, cols, ctypes.c_float(eps), native.ptr(y8), native.ptr(y8_scale),
                native.ptr(amax_in), native.ptr(amax_out), native.ptr(scale_inv_out), native.stream()
            ), 'layernorm_fwd'
        )
        return y, y8, mean, rstd
    from msamp.common.dtype import Dtypes
    from msamp.ops import cast as _c
    xf = x2.float()
    mean = xf.mean(1)
    var = xf.var(1, unbiased=False)
    rstd = torch.rsqrt(var + eps)
    yf = (xf - mean[:, None]) * rstd[:, None] * weight.float()
    if bias is not None:
        yf = yf + bias.float()
    y = yf.to(x2.dtype)
    y8 = None
    if amax_out is not None:
        _c.amax(y, out=amax_out)
    if want_y8:
        y8 = _c.cast_to_fp8(y, Dtypes.kfloat8_e4m3, y8_scale, scale_inv_out=scale_inv_out, amax_in=amax_in)
    return (y if want_y else None), y8, mean, rstd


def layer_norm_bwd_raw(dy2, x2, weight, mean, rstd, has_bias, dres=None, amax_out=None):
    """LayerNorm backward without autograd: returns ``(dx, dgamma, dbeta or None)``.

    ``dres`` (same shape and dtype as ``x2``) is added to ``dx`` in the same pass - the gradient that reaches the
    input through the skip connection around the normalised branch; ``amax_out`` receives ``max|dx|``.
    """
    rows, cols = x2.shape
    if x2.is_cuda:
        dx = torch.empty_like(x2)
        dgamma = torch.empty_like(weight)
        dbeta = torch.empty_like(weight) if has_bias else None
        nparts = native.lib().msamp_layernorm_bwd_parts()
        part = torch.empty(nparts * 2 * cols, dtype=torch.float32, device=x2.device)
        native.check(
            native.lib().msamp_layernorm_bwd_ex(
                native.ptr(dy2), native.ptr(x2), native.ptr(weight), native.dt(x2.dtype), native.dt(weight.dtype), native.ptr(mean),
                native.ptr(rstd), native.ptr(dx), native.ptr(dgamma), native.ptr(dbeta), native.ptr(part), rows, cols, native.ptr(dres),
                native.ptr(amax_out), native.stream()
            ), 'layernorm_bwd'
        )
        return dx, dgamma, dbeta
    from msamp.ops import cast as _c
    xh = (x2.float() - mean[:, None]) * rstd[:, None]
    d = dy2.float()
    gd = d * weight.float()
    m1 = gd.mean(1, keepdim=True)
    m2 = (gd * xh).mean(1, keepdim=True)
    dxf = rstd[:, None] * (gd - m1 - xh * m2)
    if dres is not None:
        dxf = dxf + dres.float()
    dx = dxf.to(x2.dtype)
    if amax_out is not None:
        _c.amax(dx, out=amax_out)
    dgamma = (d * xh).sum(0).to(weight.dtype)
    dbeta = d.sum(0).to(weight.dtype) if has_bias else None
    return dx, dgamma, dbeta


def layer_norm(x, weight, bias=None, eps=1e-5):
    """LayerNorm over the last dimension."""
    if _use_native(x):
        cols = x.shape[-1]
        vec = 4 if x.dtype == torch.float32 else 8
        if cols % vec == 0 and cols <= native.lib().msamp_layernorm_max_cols(native.dt(x.dtype)) and weight.dtype in (
            torch.float32, torch.float16, torch.bfloat16
        ) and (bias is None or bias.dtype == weight.dtype):
            return _LayerNormFn.apply(x, weight, bias, eps)
        raise RuntimeError(f'layer_norm: unsupported shape/dtype on CUDA (cols={cols}, dtype={x.dtype}, param={weight.dtype})')
    return F.layer_norm(x.float(), (x.shape[-1], ), weight.float(), None if bias is None else bias.float(), eps).to(x.dtype)


# ---------------------------------------------------------------------------------------- GeLU
class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        y = torch.empty_like(x)
        native.check(native.lib().msamp_gelu_fwd(native.ptr(x), native.ptr(y), native.i64(x.numel()), native.dt(x.dtype), native.stream()), 'gelu_fwd')
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        native.check(
            native.lib().msamp_gelu_bwd(native.ptr(x), native.ptr(dy), native.ptr(dx), native.i64(x.numel()), native.dt(x.dtype), native.stream()),
            'gelu_bwd'
        )
        return dx


def gelu(x):
    """GeLU, tanh form."""
    if _use_native(x):
        return _GeluFn.apply(x)
    return F.gelu(x.float(), approximate='tanh').to(x.dtype)


# ---------------------------------------------------------------------------------------- attention
def _attn_entry(d, which):
    """Native entry point for head size ``d``: the tcgen05 kernels for 128 (``MSAMP_ATTN_IMPL=mma`` keeps the
    mma.sync kernels, which always serve head size 64)."""
    tc = d == 128 and os.environ.get('MSAMP_ATTN_IMPL', 'tc') != 'mma'
    return getattr(native.lib(), f'msamp_attention_{"tc_" if tc else ""}{which}')


def _strides(t):
    # t is a [B, S, nh, d] view; kernel wants element strides (batch, seq, head)
    assert t.stride(3) == 1
    return [t.stride(0), t.stride(1), t.stride(2)]


class _AttentionFn(torch.autograd.Function):
    """Inputs are [B, S, nh, d] bf16 views (arbitrary batch/seq/head strides); output is contiguous [B, S, nh, d]."""
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, grad_layout):
        B, S, nh, d = q.shape
        o = torch.empty((B, S, nh, d), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, nh, S), dtype=torch.float32, device=q.device)
        st = _strides(q) + _strides(k) + _strides(v) + _strides(o) + [0] * 12
        native.check(
            _attn_entry(d, 'fwd')(
                native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(o), native.ptr(lse), _i64x24(*st), B, nh, S, d,
                ctypes.c_float(scale), int(causal), native.stream()
            ), 'attention_fwd'
        )
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale, ctx.grad_layout = causal, scale, grad_layout
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        B, S, nh, d = q.shape
        if d_o.stride(3) != 1:
            d_o = d_o.contiguous()
        if ctx.grad_layout == 'packed':
            # one [B, S, 3, nh, d] buffer so that the gradient of a fused QKV projection needs no concatenation
            dqkv = torch.empty((B, S, 3, nh, d), dtype=q.dtype, device=q.device)
            dq, dk, dv = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
        else:
            dq, dk, dv = torch.empty_like(o), torch.empty_like(o), torch.empty_like(o)
        delta = torch.empty((B, nh, S), dtype=torch.float32, device=q.device)
        st = _strides(q) + _strides(k) + _strides(v) + _strides(o) + _strides(d_o) + _strides(dq) + _strides(dk) + _strides(dv)
        native.check(
            _attn_entry(d, 'bwd')(
                native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(o), native.ptr(lse), native.ptr(d_o), native.ptr(dq),
                native.ptr(dk), native.ptr(dv), native.ptr(delta), _i64x24(*st), B, nh, S, d, ctypes.c_float(ctx.scale), int(ctx.causal),
                native.stream()
            ), 'attention_bwd'
        )
        return dq, dk, dv, None, None, None


class _AttentionPackedFn(torch.autograd.Function):
    """Attention on a fused ``[B, S, 3, heads, d]`` QKV tensor; the gradient comes back in the same packed layout.

    Taking the packed tensor as the one autograd input (instead of three ``select`` views of it) keeps
    autograd from materialising three zero-filled full-size gradients and adding them up.
    """
    @staticmethod
    def forward(ctx, qkv, causal, scale):
        B, S, _, nh, d = qkv.shape
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        o = torch.empty((B, S, nh, d), dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty((B, nh, S), dtype=torch.float32, device=qkv.device)
        st = _strides(q) + _strides(k) + _strides(v) + _strides(o) + [0] * 12
        native.check(
            _attn_entry(d, 'fwd')(
                native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(o), native.ptr(lse), _i64x24(*st), B, nh, S, d,
                ctypes.c_float(scale), int(causal), native.stream()
            ), 'attention_fwd'
        )
        ctx.save_for_backward(qkv, o, lse)
        ctx.causal, ctx.scale = causal, scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        qkv, o, lse = ctx.saved_tensors
        B, S, _, nh, d = qkv.shape
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        if d_o.stride(3) != 1 or any(s % 8 for s in d_o.stride()[:3]):
            d_o = d_o.contiguous()
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
        delta = torch.empty((B, nh, S), dtype=torch.float32, device=qkv.device)
        st = _strides(q) + _strides(k) + _strides(v) + _strides(o) + _strides(d_o) + _strides(dq) + _strides(dk) + _strides(dv)
        native.check(
            _attn_entry(d, 'bwd')(
                native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(o), native.ptr(lse), native.ptr(d_o), native.ptr(dq),
                native.ptr(dk), native.ptr(dv), native.ptr(delta), _i64x24(*st), B, nh, S, d, ctypes.c_float(ctx.scale), int(ctx.causal),
                native.stream()
            ), 'attention_bwd'
        )
        return dqkv, None, None


def attention_qkv_fwd_raw(qkv, causal=True, scale=None):
    """Self-attention forward without autograd on a packed ``[B, S, 3, heads, d]`` tensor: returns ``(o [B,S,heads,d], lse or None)``."""
    B, S, _, nh, d = qkv.shape
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if _use_native(qkv):
        if qkv.dtype != torch.bfloat16 or d not in (64, 128) or not qkv.is_contiguous() or qkv.data_ptr() % 16:
            raise RuntimeError(f'attention_qkv: CUDA kernel needs contiguous bf16 with head_dim 64/128 (got {qkv.dtype}, {d})')
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        o = torch.empty((B, S, nh, d), dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty((B, nh, S), dtype=torch.float32, device=qkv.device)
        st = _strides(q) + _strides(k) + _strides(v) + _strides(o) + [0] * 12
        native.check(
            _attn_entry(d, 'fwd')(
                native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(o), native.ptr(lse), _i64x24(*st), B, nh, S, d,
                ctypes.c_float(scale), int(causal), native.stream()
            ), 'attention_fwd'
        )
        return o, lse
    with torch.no_grad():
        return attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal=causal, scale=scale), None


def attention_qkv_bwd_raw(qkv, o, lse, d_o, causal=True, scale=None):
    """Gradient of :func:`attention_qkv_fwd_raw` with respect to the packed ``qkv`` (same layout)."""
    B, S, _, nh, d = qkv.shape
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if _use_native(qkv):
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        if d_o.stride(3) != 1 or any(s % 8 for s in d_o.stride()[:3]):
            d_o = d_o.contiguous()
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
        delta = torch.empty((B, nh, S), dtype=torch.float32, device=qkv.device)
        st = _strides(q) + _strides(k) + _strides(v) + _strides(o) + _strides(d_o) + _strides(dq) + _strides(dk) + _strides(dv)
        native.check(
            _attn_entry(d, 'bwd')(
                native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(o), native.ptr(lse), native.ptr(d_o), native.ptr(dq),
                native.ptr(dk), native.ptr(dv), native.ptr(delta), _i64x24(*st), B, nh, S, d, ctypes.c_float(scale), int(causal),
                native.stream()
            ), 'attention_bwd'
        )
        return dqkv
    with torch.enable_grad():
        leaf = qkv.detach().clone().requires_grad_(True)
        out = attention(leaf[:, :, 0], leaf[:, :, 1], leaf[:, :, 2], causal=causal, scale=scale)
        grad, = torch.autograd.grad(out, leaf, d_o)
    return grad


def attention_qkv(qkv, causal=True, scale=None):
    """Self-attention on a fused ``[B, S, 3, heads, head_dim]`` projection output; returns ``[B, S, heads, head_dim]``."""
    d = qkv.shape[-1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if _use_native(qkv):
        if qkv.dtype != torch.bfloat16 or d not in (64, 128) or not qkv.is_contiguous() or qkv.data_ptr() % 16:
            raise RuntimeError(f'attention_qkv: CUDA kernel needs contiguous bf16 with head_dim 64/128 (got {qkv.dtype}, {d})')
        return _AttentionPackedFn.apply(qkv, causal, scale)
    return attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal=causal, scale=scale)


def attention(q, k, v, causal=True, scale=None, grad_layout='separate'):
    """Softmax attention on ``[B, S, heads, head_dim]`` tensors; returns ``[B, S, heads, head_dim]``.

    ``grad_layout='packed'`` makes backward return dq/dk/dv as views of one ``[B,S,3,heads,d]`` buffer
    (use it when q, k, v are themselves views of a fused QKV tensor of that layout).
    """
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if _use_native(q):
        if q.dtype != torch.bfloat16 or d not in (64, 128):
            raise RuntimeError(f'attention: CUDA kernel supports bf16 with head_dim 64/128 (got {q.dtype}, {d})')
        for t in (q, k, v):
            if t.stride(3) != 1 or any(s % 8 for s in t.stride()[:3]) or t.data_ptr() % 16:
                raise RuntimeError('attention: operands must have unit inner stride and 16-byte aligned rows')
        return _AttentionFn.apply(q, k, v, causal, scale, grad_layout)
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        S = q.shape[1]
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device=q.device).triu(1), float('-inf'))
    out = torch.softmax(s, dim=-1) @ vf
    return out.permute(0, 2, 1, 3).to(q.dtype).contiguous()


# ---------------------------------------------------------------------------------------- cross entropy
class _XentFn(torch.autograd.Function):
    """Mean token cross-entropy; backward overwrites the logits buffer with its gradient."""
    @staticmethod
    def forward(ctx, logits, target, ignore_index):
        rows, vocab = logits.shape
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        native.check(
            native.lib().msamp_xent_fwd(
                native.ptr(logits), native.ptr(target), native.ptr(loss), native.ptr(lse), rows, vocab, native.i64(logits.stride(0)),
                native.i64(ignore_index), native.dt(logits.dtype), native.stream()
            ), 'xent_fwd'
        )
        count = (target != ignore_index).sum().clamp(min=1).float()
        ctx.save_for_backward(logits, target, lse, count)
        ctx.ignore_index = ignore_index
        return loss.sum() / count

    @staticmethod
    def backward(ctx, dloss):
        logits, target, lse, count = ctx.saved_tensors
        rows, vocab = logits.shape
        gscale = (dloss.float() / count).reshape(1).contiguous()
        native.check(
            native.lib().msamp_xent_bwd(
                native.ptr(logits), native.ptr(target), native.ptr(lse), native.ptr(gscale), rows, vocab, native.i64(logits.stride(0)),
                native.i64(ctx.ignore_index), native.dt(logits.dtype), native.stream()
            ), 'xent_bwd'
        )
        return logits, None, None


def cross_entropy(logits, target, ignore_index=-100):
    """Mean cross-entropy of ``logits [rows, vocab]`` against ``target [rows]`` (int64).

    On CUDA the backward pass reuses the logits buffer for the gradient, so ``logits`` must not be
    read again after ``backward``.
    """
    if _use_native(logits):
        if logits.stride(1) != 1:
            logits = logits.contiguous()
        return _XentFn.apply(logits, target.contiguous(), ignore_index)
    return F.cross_entropy(logits.float(), target, ignore_index=ignore_index)
