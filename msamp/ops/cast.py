"""Cast family: amax, quantise to FP8 (optionally with a transposed copy), dequantise, transpose.

CUDA tensors run the kernels of ``csrc/cast.cu``; CPU tensors run an emulation that clamps to the
format's finite range before converting through ``torch.float8_*`` (the hardware conversion
saturates, torch's does not).  Both honour the same contract:

* ``out = saturate(x * scale)`` in round-to-nearest-even;
* ``amax`` receives ``max|x|`` with NaN counted as ``+inf``.
"""
import ctypes

import torch

from msamp.common.dtype import Dtypes, Floating
from msamp.ops import native

_F8 = Dtypes.qtype_to_float8
_INF = float('inf')
_counters = {}


def _counter(device):
    """Zeroed scratch word used by the amax kernel's last-block election (one per device and stream)."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    c = _counters.get(key)
    if c is None:
        c = torch.zeros(1, dtype=torch.int32, device=device)
        _counters[key] = c
    return c


def compute_scale(amax, scale, fp_max, margin=0):
    """Power-of-two scale rule on tensors (any device); see ``ScalingMeta.compute_scaling_factor``."""
    amax = amax.float()
    exp = torch.floor(torch.log2(fp_max / amax)) - margin
    exp = exp.clamp(-126, 126)
    sf = torch.exp2(exp)
    ok = (amax > 0) & torch.isfinite(amax)
    return torch.where(ok, sf, scale)


def amax(x, out=None):
    """``max|x|`` as a 0-d fp32 tensor (NaN → inf). Writes into ``out`` when given."""
    if x.is_cuda:
        if out is None:
            out = torch.empty((), dtype=torch.float32, device=x.device)
        x = x.contiguous()
        native.check(
            native.lib().msamp_amax(
                native.ptr(x), native.i64(x.numel()), native.dt(x.dtype), native.ptr(out), None, None, ctypes.c_float(0), 0,
                ctypes.c_float(1), None, native.stream()
            ), 'amax'
        )
        return out
    if x.numel() == 0:
        val = torch.zeros((), dtype=torch.float32)
    else:
        val = torch.nan_to_num(x.detach().float().abs().max(), nan=_INF, posinf=_INF)
    if out is not None:
        out.copy_(val)
        return out
    return val


def amax_and_scale(x, amax_out, scale, scale_inv, qtype, margin=0, prescale=1.0):
    """In-time scaling in one pass over ``x``: amax → scale (→ scale_inv). All outputs are 0-d fp32 tensors."""
    fp_max = Floating.qfp_max[qtype]
    if x.is_cuda:
        x = x.contiguous()
        native.check(
            native.lib().msamp_amax(
                native.ptr(x), native.i64(x.numel()), native.dt(x.dtype), native.ptr(amax_out), native.ptr(scale),
                native.ptr(scale_inv), ctypes.c_float(fp_max), int(margin), ctypes.c_float(prescale), native.ptr(_counter(x.device)),
                native.stream()
            ), 'amax_and_scale'
        )
        return
    amax(x, out=amax_out)
    scale.copy_(compute_scale(amax_out, scale, fp_max, margin) * prescale)
    scale_inv.copy_(torch.reciprocal(scale))


def _emulate_to_fp8(x, scale, qtype):
    fmax = Floating.qfp_max[qtype]
    y = x.float() * scale.float()
    y = torch.where(torch.isnan(y), y, y.clamp(-fmax, fmax))
    return y.to(_F8[qtype]).view(torch.uint8)


def cast_to_fp8(x, qtype, scale, amax_out=None, scale_inv_out=None, amax_in=None, prescale=1.0, out=None, rescale=False, act=None,
                colsum_out=None):
    """Quantise ``x`` (fp32/fp16/bf16) to FP8 bytes with the given scale.

    Optionally records ``max|x|`` in ``amax_out`` and ``1/scale`` in ``scale_inv_out`` in the same pass.
    With ``amax_in`` (a 0-d tensor already holding ``max|x|``, e.g. from a GEMM epilogue) the scale is
    first recomputed from it by the power-of-two rule, times ``prescale``, and written to ``scale``.
    With ``rescale`` as well, ``x`` is a *scaled* tensor ``x0 * s_old``: ``scale`` must hold ``1 / s_old`` and
    ``amax_in`` ``max|x0|``; the bytes are ``x0 * s_new`` with ``s_new`` from the rule, ``scale_inv_out`` receives
    ``1 / s_new`` and ``scale`` is left alone (the cast of a scaled 16-bit master weight).
    ``act='gelu'`` quantises ``gelu(x)`` (tanh form, rounded to the dtype of ``x`` first) instead of ``x``.
    ``colsum_out`` (fp32 ``[cols]``, zero on entry) receives the column sums of a 2-D ``x`` from the same pass - the
    bias gradient when ``x`` is the output gradient of a linear layer.
    ``out`` (uint8, same number of elements, contiguous) receives the bytes when given.
    """
    if out is not None:
        assert out.dtype == torch.uint8 and out.numel() == x.numel() and out.is_contiguous() and out.device == x.device
    if rescale:
        assert amax_in is not None
    if colsum_out is not None:
        assert x.dim() == 2 and act is None and not rescale
        assert colsum_out.dtype == torch.float32 and colsum_out.numel() == x.shape[1] and colsum_out.is_contiguous()
    if x.is_cuda:
        x = x.contiguous()
        if out is None:
            out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
        if colsum_out is not None and (x.shape[1] * x.element_size()) % 16 == 0 and x.data_ptr() % 16 == 0 and out.data_ptr() % 8 == 0:
            native.check(
                native.lib().msamp_cast_to_fp8_colsum(
                    native.ptr(x), x.shape[0], x.shape[1], native.dt(x.dtype), native.ptr(out), native.fmt(qtype), native.ptr(scale),
                    native.ptr(amax_out), native.ptr(scale_inv_out), native.ptr(colsum_out), native.ptr(amax_in), native.stream()
                ), 'cast_to_fp8_colsum'
            )
            return out
        native.check(
            native.lib().msamp_cast_to_fp8_ex(
                native.ptr(x), native.i64(x.numel()), native.dt(x.dtype), native.ptr(out), native.fmt(qtype), native.ptr(scale),
                native.ptr(amax_out), native.ptr(scale_inv_out), native.ptr(amax_in), ctypes.c_float(prescale), int(bool(rescale)),
                1 if act == 'gelu' else 0, native.stream()
            ), 'cast_to_fp8'
        )
        if colsum_out is not None:
            colsum_out.add_(x.sum(0, dtype=torch.float32))
        return out
    if act == 'gelu':
        x = torch.nn.functional.gelu(x.float(), approximate='tanh').to(x.dtype)
    if rescale:
        new_scale = compute_scale(amax_in, torch.ones_like(scale), Floating.qfp_max[qtype])
        if scale_inv_out is not None:
            torch.reciprocal(new_scale, out=scale_inv_out)
        scale = new_scale * scale
    else:
        if amax_in is not None:
            scale.copy_(compute_scale(amax_in, scale, Floating.qfp_max[qtype]) * torch.where(
                (amax_in > 0) & torch.isfinite(amax_in), prescale, 1.0))
        if scale_inv_out is not None:
            torch.reciprocal(scale, out=scale_inv_out)
    if amax_out is not None:
        amax(x, out=amax_out)
    if colsum_out is not None:
        colsum_out.add_(x.sum(0, dtype=torch.float32))
    res = _emulate_to_fp8(x, scale, qtype)
    if out is not None:
        out.copy_(res.view_as(out))
        return out
    return res


def cast_transpose_fp8(x, qtype, scale, amax_out=None, need_rowmajor=True, scale_inv_out=None, amax_in=None, colsum_out=None):
    """Quantise a 2-D tensor and also produce its transpose. Returns ``(out or None, out_t)``.

    ``colsum_out`` (fp32 ``[cols]``, zero on entry) receives the column sums of ``x`` from the same pass - the bias
    gradient when ``x`` is the output gradient of a linear layer.

    With ``amax_in`` the input is a *scaled* tensor ``x * s_old``: ``scale`` must hold ``1 / s_old`` and ``amax_in``
    ``max|x|``; the kernel derives ``s_new`` from the amax, multiplies by ``s_new / s_old`` and writes ``1 / s_new`` to
    ``scale_inv_out`` - all in the one launch.
    """
    assert x.dim() == 2
    rows, cols = x.shape
    if x.is_cuda:
        x = x.contiguous()
        out = torch.empty((rows, cols), dtype=torch.uint8, device=x.device) if need_rowmajor else None
        out_t = torch.empty((cols, rows), dtype=torch.uint8, device=x.device)
        if colsum_out is None:
            native.check(
                native.lib().msamp_cast_transpose_fp8(
                    native.ptr(x), rows, cols, native.dt(x.dtype), native.ptr(out), native.ptr(out_t), native.fmt(qtype),
                    native.ptr(scale), native.ptr(amax_out), native.ptr(scale_inv_out), native.ptr(amax_in), native.stream()
                ), 'cast_transpose_fp8'
            )
        else:
            assert colsum_out.dtype == torch.float32 and colsum_out.numel() == cols and colsum_out.is_contiguous()
            native.check(
                native.lib().msamp_cast_transpose_fp8_colsum(
                    native.ptr(x), rows, cols, native.dt(x.dtype), native.ptr(out), native.ptr(out_t), native.fmt(qtype),
                    native.ptr(scale), native.ptr(amax_out), native.ptr(scale_inv_out), native.ptr(amax_in), native.ptr(colsum_out),
                    native.stream()
                ), 'cast_transpose_fp8_colsum'
            )
        return out, out_t
    if amax_in is not None:
        new_scale = compute_scale(amax_in, torch.ones_like(scale), Floating.qfp_max[qtype])
        if scale_inv_out is not None:
            torch.reciprocal(new_scale, out=scale_inv_out)
        scale = new_scale * scale
    elif scale_inv_out is not None:
        torch.reciprocal(scale, out=scale_inv_out)
    if amax_out is not None:
        amax(x, out=amax_out)
    if colsum_out is not None:
        colsum_out.add_(x.sum(0, dtype=torch.float32))
    out = _emulate_to_fp8(x, scale, qtype)
    return (out if need_rowmajor else None), out.t().contiguous()


def transpose_fp8(x, out=None):
    """Byte transpose of a 2-D FP8 payload (into ``out``, a contiguous ``[cols, rows]`` tensor, when given)."""
    assert x.dim() == 2
    rows, cols = x.shape
    if out is not None:
        assert out.shape == (cols, rows) and out.is_contiguous() and out.dtype == x.dtype
    if x.is_cuda:
        x = x.contiguous()
        if out is None:
            out = torch.empty((cols, rows), dtype=x.dtype, device=x.device)
        native.check(native.lib().msamp_transpose_fp8(native.ptr(x), rows, cols, native.ptr(out), native.stream()), 'transpose_fp8')
        return out
    if out is not None:
        out.copy_(x.t())
        return out
    return x.t().contiguous()


def cast_from_fp8(x, qtype, scale_inv, out_dtype):
    """Dequantise FP8 bytes: ``float(x) * scale_inv`` rounded to ``out_dtype``."""
    if x.is_cuda:
        x = x.contiguous()
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        native.check(
            native.lib().msamp_cast_from_fp8(
                native.ptr(x), native.i64(x.numel()), native.fmt(qtype), native.ptr(scale_inv), native.ptr(out), native.dt(out_dtype),
                native.stream()
            ), 'cast_from_fp8'
        )
        return out
    return (x.view(torch.uint8).view(_F8[qtype]).float() * scale_inv.float()).to(out_dtype)


def update_scales(amax_flat, scale, scale_inv, qtype, margin=0, amax_stride=1):
    """Vectorised scale rule over ``n`` metas stored in flat buffers."""
    fp_max = Floating.qfp_max[qtype]
    n = scale.numel()
    if scale.is_cuda:
        native.check(
            native.lib().msamp_update_scales(
                native.ptr(amax_flat), native.i64(amax_stride), native.ptr(scale), native.ptr(scale_inv), n, ctypes.c_float(fp_max),
                int(margin), native.stream()
            ), 'update_scales'
        )
        return
    a = amax_flat.reshape(n, -1)[:, 0] if amax_flat.numel() != n else amax_flat.reshape(n)
    scale.copy_(compute_scale(a, scale.reshape(n), fp_max, margin).view_as(scale))
    scale_inv.copy_(torch.reciprocal(scale))


def roll_windows(amaxs, scales, qtype, margin=0, bad_out=None):
    """Delayed-scaling bookkeeping for all metas of one kind in a single launch.

    ``amaxs`` is ``[n, window]`` fp32 and ``scales`` ``[n]`` fp32 on one device: a non-finite newest
    amax is dropped, the scale is recomputed from the window maximum, and the window moves one slot.
    ``bad_out`` (optional ``[n]`` int32 on the same device) is set to 1 where a non-finite amax was
    seen.  Behaviour follows LBOptimizer._update_scaling_factors of the reference
    (msamp/optim/optimizer.py:61-108) except that step counters stay on the host.
    """
    fp_max = Floating.qfp_max[qtype]
    n, window = amaxs.shape
    if amaxs.is_cuda:
        native.check(
            native.lib().msamp_roll_windows(
                native.ptr(amaxs), native.ptr(scales), native.ptr(bad_out), n, window, ctypes.c_float(fp_max), int(margin),
                native.stream()
            ), 'roll_windows'
        )
        return
    bad = ~torch.isfinite(amaxs[:, 0])
    amaxs[bad, 0] = 0
    scales.copy_(compute_scale(amaxs.max(1).values, scales, fp_max, margin))
    amaxs.copy_(amaxs.roll(1, dims=1))
    amaxs[:, 0] = 0
    if bad_out is not None:
        bad_out.copy_(bad.to(torch.int32))
