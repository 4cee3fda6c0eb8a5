"""FP8 GEMM:  ``D[M,N] = epilogue((sa_inv * sb_inv) * A[M,K] @ B[N,K]^T)``.

On CUDA this is the tcgen05/TMEM kernel of ``csrc/gemm_fp8.cu``; on CPU the operands are
dequantised and multiplied in fp32, which is also the test oracle.

Either operand may be handed over in its transposed storage (``a_mn`` / ``b_mn``): the tensor core
reads both layouts, so callers never materialise an FP8 transpose.
"""
import ctypes
import os

import torch

from msamp.common.dtype import Dtypes
from msamp.ops import native

_F8 = Dtypes.qtype_to_float8
# MSAMP_GEMM_TILE=1|2 forces the CTA-pair or the single-CTA kernel for every call that does not choose itself; 0 lets the library choose
_DEFAULT_TILE = int(os.environ.get('MSAMP_GEMM_TILE', '0'))


class _GemmDesc(ctypes.Structure):
    """Mirror of ``MsampGemmDesc`` in csrc/gemm_fp8.cu."""
    _fields_ = [
        ('a', ctypes.c_void_p), ('b', ctypes.c_void_p), ('d', ctypes.c_void_p), ('bias', ctypes.c_void_p),
        ('residual', ctypes.c_void_p), ('gelu_src', ctypes.c_void_p), ('scale_inv_a', ctypes.c_void_p),
        ('scale_inv_b', ctypes.c_void_p), ('amax_out', ctypes.c_void_p), ('d8', ctypes.c_void_p), ('d8_scale', ctypes.c_void_p), ('d8_scale_inv_out', ctypes.c_void_p),
        ('lda', ctypes.c_int64), ('ldb', ctypes.c_int64), ('ldd', ctypes.c_int64), ('ldr', ctypes.c_int64), ('ldg', ctypes.c_int64),
        ('ld8', ctypes.c_int64),
        ('M', ctypes.c_int), ('N', ctypes.c_int), ('K', ctypes.c_int), ('a_fmt', ctypes.c_int), ('b_fmt', ctypes.c_int),
        ('d8_fmt', ctypes.c_int), ('a_mn', ctypes.c_int), ('b_mn', ctypes.c_int), ('out_dtype', ctypes.c_int),
        ('bias_dtype', ctypes.c_int), ('act', ctypes.c_int), ('max_ctas', ctypes.c_int), ('tile', ctypes.c_int), ('stats', ctypes.c_void_p),
        ('colsum', ctypes.c_void_p),
    ]


def _gelu_tanh(x):
    return torch.nn.functional.gelu(x, approximate='tanh')


def _gelu_tanh_grad(x):
    k0, k1 = 0.7978845608028654, 0.044715
    u = k0 * (x + k1 * x * x * x)
    th = torch.tanh(u)
    return 0.5 * (1.0 + th) + 0.5 * x * (1.0 - th * th) * k0 * (1.0 + 3.0 * k1 * x * x)


def _fix_operand(t):
    if t.stride(1) != 1 or t.stride(0) % 16 or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def gemm_fp8(a, a_qtype, a_scale_inv, b, b_qtype, b_scale_inv, out_dtype, bias=None, accumulate=False, out=None, amax_out=None,
             max_ctas=0, a_mn=False, b_mn=False, residual=None, gelu_src=None, act=None, out8=None, out8_qtype=None, out8_scale=None,
             out8_scale_inv_out=None, tile=0, stats=None, colsum_out=None, store_out=True):
    """Multiply FP8 byte matrices.

    Args:
        a: uint8 ``[M,K]`` (or ``[K,M]`` with ``a_mn``) holding e4m3/e5m2 bytes, last dimension contiguous.
        b: uint8 ``[N,K]`` (or ``[K,N]`` with ``b_mn``).
        a_qtype, b_qtype: their formats.
        a_scale_inv, b_scale_inv: 0-d fp32 tensors (dequantisation factors).
        out_dtype: fp32 / fp16 / bf16.
        bias: optional ``[N]`` vector added to every row.
        accumulate: add the product to the existing contents of ``out``.
        out: optional ``[M,N]`` destination (required with ``accumulate``).
        amax_out: optional 0-d fp32 tensor receiving ``max|D|`` of the stored values (``max|gelu(D)|`` with ``act='gelu'``).
        max_ctas: cap on persistent CTAs (0 = one per SM).
        residual: optional ``[M,N]`` tensor of ``out_dtype`` added to the product (a skip connection).
        gelu_src: optional ``[M,N]`` tensor ``h`` of ``out_dtype``; the product is multiplied by ``gelu'(h)``
            (the backward of a GeLU that followed the layer whose input gradient this GEMM computes).
        act: ``None`` or ``'gelu'``: which function of ``D`` ``amax_out`` and ``out8`` describe.
        out8, out8_qtype, out8_scale: optional uint8 ``[M,N]`` receiving ``quantise(act(D) * out8_scale)``;
            ``out8_scale_inv_out`` (optional) then receives ``1 / out8_scale``.
        colsum_out: optional fp32 ``[N]`` receiving the column sums of ``D`` as stored (the bias gradient when ``D`` is the
            output gradient of a biased layer); it is overwritten.
        store_out: ``False`` skips ``D`` itself (returns ``None``) when only ``amax_out`` / ``out8`` / ``colsum_out`` are wanted.
        tile: 0 = choose, 1 = CTA-pair 256x256 tiles, 2 = single-CTA tiles (CUDA only; for tests and benchmarks).
        stats: optional int64 ``[4 * CTAs]`` CUDA tensor receiving per-CTA cycle counters (producer wait, MMA wait for
            data, MMA wait for TMEM, MMA warp total) for tuning.
    """
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
    assert K == Kb, (a.shape, b.shape, a_mn, b_mn)
    if accumulate and out is None:
        raise ValueError('accumulate=True needs an output tensor')
    if accumulate and residual is not None:
        raise ValueError('accumulate and residual exclude each other')
    if not store_out:
        if out is not None or accumulate or residual is not None:
            raise ValueError('store_out=False excludes out, accumulate and residual')
        if amax_out is None and out8 is None and colsum_out is None:
            raise ValueError('store_out=False needs another output')
    elif out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    else:
        assert out.shape == (M, N) and out.dtype == out_dtype and out.stride(1) == 1
    if colsum_out is not None:
        assert colsum_out.shape == (N, ) and colsum_out.dtype == torch.float32 and colsum_out.is_contiguous()
    if accumulate:
        residual = out
    for t in (residual, gelu_src):
        if t is not None:
            assert t.shape == (M, N) and t.dtype == out_dtype and t.stride(1) == 1
    if out8 is not None:
        assert out8.shape == (M, N) and out8.dtype == torch.uint8 and out8.stride(1) == 1 and out8_scale is not None
    if a.is_cuda:
        a, b = _fix_operand(a), _fix_operand(b)
        if K % 16 and not (a_mn and b_mn):
            if a_mn or b_mn:
                raise ValueError('K must be a multiple of 16 when one operand is K-major and the other is not')
            pad = 16 - K % 16
            a, b = torch.nn.functional.pad(a, (0, pad)), torch.nn.functional.pad(b, (0, pad))
            K += pad
        if amax_out is not None:
            amax_out.zero_()
        if colsum_out is not None:
            colsum_out.zero_()
        g = _GemmDesc()
        g.a, g.b, g.d = a.data_ptr(), b.data_ptr(), (out.data_ptr() if out is not None else None)
        g.colsum = colsum_out.data_ptr() if colsum_out is not None else None
        g.bias = bias.data_ptr() if bias is not None else None
        g.residual = residual.data_ptr() if residual is not None else None
        g.gelu_src = gelu_src.data_ptr() if gelu_src is not None else None
        g.scale_inv_a, g.scale_inv_b = a_scale_inv.data_ptr(), b_scale_inv.data_ptr()
        g.amax_out = amax_out.data_ptr() if amax_out is not None else None
        g.d8 = out8.data_ptr() if out8 is not None else None
        g.d8_scale = out8_scale.data_ptr() if out8 is not None else None
        g.d8_scale_inv_out = out8_scale_inv_out.data_ptr() if (out8 is not None and out8_scale_inv_out is not None) else None
        g.lda, g.ldb, g.ldd = a.stride(0), b.stride(0), (out.stride(0) if out is not None else N)
        g.ldr = residual.stride(0) if residual is not None else 0
        g.ldg = gelu_src.stride(0) if gelu_src is not None else 0
        g.ld8 = out8.stride(0) if out8 is not None else 0
        g.M, g.N, g.K = M, N, K
        g.a_fmt, g.b_fmt = native.fmt(a_qtype), native.fmt(b_qtype)
        g.d8_fmt = native.fmt(out8_qtype) if out8 is not None else 0
        g.a_mn, g.b_mn = int(bool(a_mn)), int(bool(b_mn))
        g.out_dtype = native.dt(out_dtype)
        g.bias_dtype = native.dt(bias.dtype) if bias is not None else 0
        g.act = 1 if act == 'gelu' else 0
        g.max_ctas, g.tile = int(max_ctas), int(tile) or _DEFAULT_TILE
        g.stats = stats.data_ptr() if stats is not None else None
        native.check(native.lib().msamp_gemm_fp8_ex(ctypes.byref(g), native.stream()), 'gemm_fp8')
        return out
    af = a.view(torch.uint8).view(_F8[a_qtype]).float()
    bf = b.view(torch.uint8).view(_F8[b_qtype]).float()
    if a_mn:
        af = af.t()
    if b_mn:
        bf = bf.t()
    res = (af @ bf.t()) * (a_scale_inv.float() * b_scale_inv.float())
    if bias is not None:
        res = res + bias.float()
    if residual is not None:
        res = res + residual.float()
    if gelu_src is not None:
        res = res * _gelu_tanh_grad(gelu_src.float())
    stored = res.to(out_dtype)
    if out is not None:
        out.copy_(stored)
    if colsum_out is not None:
        colsum_out.copy_(stored.float().sum(0))
    if amax_out is not None or out8 is not None:
        w = stored.float()
        if act == 'gelu':
            w = _gelu_tanh(w).to(out_dtype).float()
        if amax_out is not None:
            amax_out.copy_(torch.nan_to_num(w.abs().max(), nan=float('inf')))
        if out8 is not None:
            from msamp.ops.cast import _emulate_to_fp8
            out8.copy_(_emulate_to_fp8(w, out8_scale, out8_qtype))
            if out8_scale_inv_out is not None:
                torch.reciprocal(out8_scale, out=out8_scale_inv_out)
    return out
