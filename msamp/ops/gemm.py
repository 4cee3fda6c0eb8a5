"""FP8 GEMM:  ``D[M,N] = (sa_inv * sb_inv) * A[M,K] @ B[N,K]^T (+ bias) (+ D)``.

On CUDA this is the tcgen05/TMEM kernel of ``csrc/gemm_fp8.cu``; on CPU the operands are
dequantised and multiplied in fp32, which is also the test oracle.
"""
import torch

from msamp.common.dtype import Dtypes
from msamp.ops import native

_F8 = Dtypes.qtype_to_float8


def _pad_k(t, k_pad):
    if k_pad == 0:
        return t
    return torch.nn.functional.pad(t, (0, k_pad))


def gemm_fp8(a, a_qtype, a_scale_inv, b, b_qtype, b_scale_inv, out_dtype, bias=None, accumulate=False, out=None, amax_out=None,
             max_ctas=0):
    """Multiply FP8 byte matrices ``a[M,K]`` and ``b[N,K]`` (K contiguous in both).

    Args:
        a, b: uint8 tensors holding e4m3/e5m2 bytes.
        a_qtype, b_qtype: their formats.
        a_scale_inv, b_scale_inv: 0-d fp32 tensors (dequantisation factors).
        out_dtype: fp32 / fp16 / bf16.
        bias: optional ``[N]`` vector added to every row.
        accumulate: add the product to the existing contents of ``out``.
        out: optional ``[M,N]`` destination (required with ``accumulate``).
        amax_out: optional 0-d fp32 tensor receiving ``max|D|`` (fused into the epilogue on CUDA).
        max_ctas: cap on persistent CTAs (0 = one per SM).
    """
    assert a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1], (a.shape, b.shape)
    M, K = a.shape
    N = b.shape[0]
    if accumulate and out is None:
        raise ValueError('accumulate=True needs an output tensor')
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    else:
        assert out.shape == (M, N) and out.dtype == out_dtype and out.stride(1) == 1
    if a.is_cuda:
        if a.stride(1) != 1 or a.stride(0) % 16 or a.data_ptr() % 16:
            a = a.contiguous()
        if b.stride(1) != 1 or b.stride(0) % 16 or b.data_ptr() % 16:
            b = b.contiguous()
        if K % 16:
            pad = 16 - K % 16
            a, b = _pad_k(a, pad), _pad_k(b, pad)
            K += pad
        if amax_out is not None:
            amax_out.zero_()
        native.check(
            native.lib().msamp_gemm_fp8(
                native.ptr(a), native.ptr(b), native.ptr(out), M, N, K, native.i64(a.stride(0)), native.i64(b.stride(0)),
                native.i64(out.stride(0)), native.fmt(a_qtype), native.fmt(b_qtype), native.dt(out_dtype), native.ptr(a_scale_inv),
                native.ptr(b_scale_inv), native.ptr(bias), native.dt(bias.dtype) if bias is not None else 0, int(bool(accumulate)),
                native.ptr(amax_out), int(max_ctas), native.stream()
            ), 'gemm_fp8'
        )
        return out
    af = a.view(torch.uint8).view(_F8[a_qtype]).float()
    bf = b.view(torch.uint8).view(_F8[b_qtype]).float()
    res = (af @ bf.t()) * (a_scale_inv.float() * b_scale_inv.float())
    if bias is not None:
        res = res + bias.float()
    if accumulate:
        res = res + out.float()
    out.copy_(res.to(out_dtype))
    if amax_out is not None:
        amax_out.copy_(torch.nan_to_num(out.float().abs().max(), nan=float('inf')))
    return out
