"""Simulated FP4 quantisation of bf16 tensors and the DGE derivative.

The tensor stays in bf16; only its values are snapped to what a 4-bit format could hold after a
power-of-two scale (per tensor, per channel = column, or per token = row).  ``e2m1`` uses the
value table {0, ±.5, ±1, ±1.5, ±2, ±3, ±4, ±6}; ``e1m2`` is uniform, emulated by rounding after
scaling to ±7.  (reference: msamp/operators/fp4_quantize/fp4_quantize.py:17-186)
"""
import torch

from msamp.common.tensor import ScalingMeta
from msamp.ops import arith as _a


class FP4_QUANTIZER:
    """Namespace of static FP4-simulation helpers."""
    @staticmethod
    def apply_DGE_item(input_tensor, k=5.0, power_clamp_max=3.0):
        """Element-wise derivative of the differentiable e2m1 quantiser (bf16 in, bf16 out)."""
        if input_tensor.dtype != torch.bfloat16:
            raise ValueError('The input tensor is not in bfloat16.')
        return _a.fp4_dge(input_tensor.contiguous(), float(k), float(power_clamp_max))

    @staticmethod
    def _apply_quantile_clipping(input, clip_threshold=0.99, channel_wise=False, token_wise=False, return_residual=False):
        """Clamp to the [1-q, q] quantiles (global, per column or per row); optionally return what was cut off."""
        if channel_wise or token_wise:
            dim = 0 if channel_wise else 1
            ordered = torch.sort(input, dim=dim).values
            n = ordered.size(dim)
            lo = ordered.narrow(dim, int((1 - clip_threshold) * n), 1)
            hi = ordered.narrow(dim, int(clip_threshold * n), 1)
        else:
            ordered = torch.sort(input.float().reshape(-1)).values
            n = ordered.numel()
            lo = ordered[int((1 - clip_threshold) * n)]
            hi = ordered[int(clip_threshold * n)]
        out = torch.clamp(input, min=lo.to(input.dtype), max=hi.to(input.dtype)).to(input.dtype)
        return (out, input - out) if return_residual else (out, None)

    @staticmethod
    def quantize_simulate_fp4_in_bf16(
        input_tensor, format='e1m2', nan_existed=False, channel_wise=False, token_wise=False, outlier_clip=False, clip_threshold=0.99,
        residual_compensation=False, return_scaled_input_for_bwd=False
    ):
        """Return ``input_tensor`` snapped to simulated FP4 values (still bf16); see the module docstring."""
        if input_tensor.dtype != torch.bfloat16:
            raise ValueError('The input tensor is not in bfloat16.')
        if channel_wise and token_wise:
            raise AssertionError('channel_wise and token_wise cannot be True at the same time.')
        if format not in ('e2m1', 'e1m2'):
            raise ValueError(f'unknown FP4 format {format}')
        x = input_tensor.contiguous()
        shape = x.shape
        if (channel_wise or token_wise) and x.dim() != 2:
            x = x.reshape(-1, shape[-1])
        residual = None
        if outlier_clip:
            x, residual = FP4_QUANTIZER._apply_quantile_clipping(x, clip_threshold, channel_wise, token_wise, residual_compensation)
        if channel_wise:
            amax = x.abs().amax(dim=0, keepdim=True)
        elif token_wise:
            amax = x.abs().amax(dim=1, keepdim=True)
        else:
            amax = x.abs().max()
        fp_max = 6.0 if format == 'e2m1' else 7.0
        sf = ScalingMeta.compute_scaling_factor(amax, torch.ones_like(amax, dtype=torch.float32), fp_max, 0).to(x.dtype)
        scaled = x * sf
        out = _a.fp4_quantize_e2m1(scaled) if format == 'e2m1' else torch.round(scaled)
        out = out / sf
        if residual_compensation and residual is not None:
            out = out + residual
        out.requires_grad = input_tensor.requires_grad
        if out.shape != shape:
            out = out.view(shape)
            scaled = scaled.view(shape)
        if return_scaled_input_for_bwd:
            return out, scaled
        return out
