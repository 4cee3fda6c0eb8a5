"""FP8 linear: autograd function and the ``torch.nn.functional.linear`` override.

Data flow of one linear (shapes: x ``[T,K]``, W ``[N,K]``, y ``[T,N]``).  The tcgen05 GEMM reads an operand either
K-major or MN-major, so x, W and dy are quantised once, in the layout they already have, and no FP8
transpose is ever written:

  forward   x  --cast(e4m3, meta 'input')-->  x8 [T,K]   (kept for backward)
            W  --cast(e4m3), cached until the weight changes-->  W8 [N,K]
            y  = x8 · W8ᵀ  (+ bias, + residual in the epilogue)
  backward  dy --cast(e5m2, meta 'ograd'; the bias gradient = column sums of dy falls out of the same pass)--> dy8 [T,N]
            dx = dy8 · W8           (W8 read as the MN-major B operand)
            dW = dy8ᵀ · x8          (both read MN-major) with max|dW| reduced in the epilogue
            dW --cast(e4m3, meta 'wgrad', scale from that amax [MAX-reduced over the DP group])--> ScalingTensor
            delivered through ``weight.backward_grad_update`` (not through autograd)

Semantics follow the reference's _FP8GemmFunction and F.linear wrapper (msamp/nn/functional.py:16-194):
formats, window sizes, gradient accumulation in high precision, FP8-DDP and FSDP special cases.
"""
import torch
import torch.distributed as dist
import torch.nn.functional as F

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingTensor, TypeCast
from msamp.common.utils.dist import DistUtil
from msamp.nn.state import model_state
from msamp.nn.parameter import ScalingParameter
from msamp.ops import cast as _k
from msamp.ops import gemm as _g

E4M3, E5M2 = Dtypes.kfloat8_e4m3, Dtypes.kfloat8_e5m2


def _bump_version(t):
    try:
        torch.autograd.graph.increment_version(t)
    except Exception:    # pragma: no cover - very old torch
        pass


def weight_fp8_pair(weight):
    """FP8 copies ``(W8 [N,K], W8ᵀ [K,N], scale_inv)`` of a weight, cached on the parameter.

    The cache key is the identity and in-place version of ``weight.value`` and of its ``scale_inv``,
    so any optimizer step, ``copy_``, ``cast_`` or checkpoint load invalidates it.
    """
    val = weight.value
    key = (val.data_ptr(), val._version, weight.meta.scale_inv._version, weight.meta.scale_inv.data_ptr())
    cache = getattr(weight, '_fp8_cache', None)
    if cache is not None and cache[0] == key:
        return cache[1], cache[2], cache[3]
    w2d = val.reshape(-1, val.shape[-1])
    if Dtypes.is_fp8_qtype(weight.meta.qtype):
        if weight.meta.qtype != E4M3:
            raise TypeError('FP8 weights must be e4m3')
        w8 = w2d
        w8t = _k.transpose_fp8(w2d)
        sinv = weight.meta.scale_inv
    else:
        # Scaled 16-bit weight: value == w * s_w. Quantise with the scale implied by the stored
        # amax of w, expressed relative to the stored payload.
        meta = weight.meta
        sinv = torch.empty_like(meta.scale_inv)
        w8, w8t = _k.cast_transpose_fp8(w2d, E4M3, meta.scale_inv, scale_inv_out=sinv, amax_in=meta.amax[0])
    weight._fp8_cache = (key, w8, w8t, sinv)
    return w8, w8t, sinv


def weight_fp8(weight):
    """FP8 copy ``(W8 [N,K], scale_inv)`` of a weight in its own layout, cached on the parameter.

    An e4m3 weight is used as it is; a scaled 16-bit weight (``value == w * s_w``) is quantised with the
    scale implied by the stored amax of ``w``.  The cache key is the identity and in-place version of
    ``weight.value`` and of its ``scale_inv``, so any optimizer step, ``copy_``, ``cast_`` or checkpoint
    load invalidates it.
    """
    val = weight.value
    w2d = val.reshape(-1, val.shape[-1])
    if Dtypes.is_fp8_qtype(weight.meta.qtype):
        if weight.meta.qtype != E4M3:
            raise TypeError('FP8 weights must be e4m3')
        return w2d, weight.meta.scale_inv
    key = (val.data_ptr(), val._version, weight.meta.scale_inv._version, weight.meta.scale_inv.data_ptr())
    cache = getattr(weight, '_fp8_cache1', None)
    if cache is not None and cache[0] == key:
        return cache[1], cache[2]
    meta = weight.meta
    sinv = torch.empty_like(meta.scale_inv)
    w8 = _k.cast_to_fp8(w2d, E4M3, meta.scale_inv, scale_inv_out=sinv, amax_in=meta.amax[0], rescale=True)
    weight._fp8_cache1 = (key, w8, sinv)
    weight._wants_fp8_copy = True    # the fused Adam step will deliver the copy of the updated weight (msamp/optim/adamw.py)
    return w8, sinv


def _tma_ok(t):
    """A 2-D byte matrix the GEMM can read MN-major: contiguous rows whose pitch and base are multiples of 16 bytes."""
    return t.stride(1) == 1 and t.stride(0) % 16 == 0 and t.data_ptr() % 16 == 0


def gemm_dgrad(dy8, dy_sinv, w8, w_sinv, out_dtype, **kw):
    """``dx[T,K] = dy8[T,N] · W8[N,K]``: the weight is read as stored (MN-major B).  Shapes the TMA cannot
    address that way (pitch not a multiple of 16 bytes) fall back to a transposed copy of the weight."""
    if _tma_ok(w8) and dy8.shape[1] % 16 == 0:
        return _g.gemm_fp8(dy8, E5M2, dy_sinv, w8, E4M3, w_sinv, out_dtype, b_mn=True, **kw)
    return _g.gemm_fp8(dy8, E5M2, dy_sinv, _k.transpose_fp8(w8), E4M3, w_sinv, out_dtype, **kw)


def gemm_wgrad(dy8, dy_sinv, x8, x_sinv, out_dtype, **kw):
    """``dW[N,K] = dy8[T,N]ᵀ · x8[T,K]``: both operands are read as stored (MN-major A and B)."""
    if _tma_ok(dy8) and _tma_ok(x8):
        return _g.gemm_fp8(dy8, E5M2, dy_sinv, x8, E4M3, x_sinv, out_dtype, a_mn=True, b_mn=True, **kw)
    return _g.gemm_fp8(_k.transpose_fp8(dy8), E5M2, dy_sinv, _k.transpose_fp8(x8), E4M3, x_sinv, out_dtype, **kw)


class _FP8GemmFunction(torch.autograd.Function):
    """y = x · Wᵀ (+ bias) with FP8 operands; weight gradient delivered out of band."""
    @staticmethod
    def forward(ctx, input, weight, metas, dtype_holder, bias=None):
        fsdp_weight = isinstance(weight, torch.Tensor) and hasattr(weight, '_meta')
        if fsdp_weight:
            # Flat fp32 FSDP parameter carrying e4m3 bytes (see msamp.fsdp): reinterpret in place.
            raw = weight.view(torch.uint8).reshape(-1)
            if weight._padded:
                raw = raw[:raw.numel() - weight._padded]
            flat_param = weight
            weight = ScalingParameter(ScalingTensor(raw.view(weight._original_shape), weight._meta))
            weight._flat_param = flat_param
        ctx.return_wgrad = fsdp_weight
        model_state.check_metas_in_flat(metas)
        out_dtype = dtype_holder.dtype
        need_wgrad = weight.requires_grad and ctx.needs_input_grad[3]    # the holder tells whether grad mode is on
        in_meta = metas['input']

        x = input.contiguous()
        record = TypeCast._prepare_scale(x, in_meta, sync=False)
        amax_out = in_meta.amax[0] if record else None
        sinv_out = in_meta.scale_inv if record else None
        x8 = _k.cast_to_fp8(x, E4M3, in_meta.scale, amax_out, scale_inv_out=sinv_out)
        x_sinv = in_meta.scale_inv.clone()    # the meta may be reused before backward runs

        w8, w_sinv = weight_fp8(weight)
        out = _g.gemm_fp8(x8, E4M3, x_sinv, w8, E4M3, w_sinv, out_dtype, bias=bias)

        ctx.metas = metas
        ctx.weight = weight
        ctx.x8, ctx.x_sinv = (x8 if need_wgrad else None), x_sinv
        ctx.w8, ctx.w_sinv = w8, w_sinv
        ctx.out_dtype = out_dtype
        ctx.input_requires_grad = input.requires_grad
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return out

    @staticmethod
    def backward(ctx, output_grad):
        dy = output_grad.contiguous()
        metas = ctx.metas
        og_meta, wg_meta = metas['ograd'], metas['wgrad']
        weight = ctx.weight
        need_wgrad = weight.requires_grad and ctx.x8 is not None

        record = TypeCast._prepare_scale(dy, og_meta, sync=False)
        amax_out = og_meta.amax[0] if record else None
        sinv_out = og_meta.scale_inv if record else None
        dbias = None
        # the bias gradient (column sums of dy) comes out of the same pass over dy
        colsum = torch.zeros(dy.shape[1], dtype=torch.float32, device=dy.device) if (ctx.has_bias and dy.dim() == 2) else None
        dy8 = _k.cast_to_fp8(dy, E5M2, og_meta.scale, amax_out, scale_inv_out=sinv_out, colsum_out=colsum)
        if colsum is not None:
            dbias = colsum.to(ctx.bias_dtype)
        dy_sinv = og_meta.scale_inv

        dx = None
        if ctx.input_requires_grad:
            dx = gemm_dgrad(dy8, dy_sinv, ctx.w8, ctx.w_sinv, ctx.out_dtype)
        if ctx.has_bias and dbias is None:
            dbias = dy.sum(0, dtype=torch.float32).to(ctx.bias_dtype)

        wgrad_ret = None
        if need_wgrad:
            amax0 = wg_meta.amax[0]
            if weight.grad is None:
                wgrad = gemm_wgrad(dy8, dy_sinv, ctx.x8, ctx.x_sinv, ctx.out_dtype, amax_out=amax0)
            else:
                old = weight.grad.to(ctx.out_dtype)
                wgrad = gemm_wgrad(dy8, dy_sinv, ctx.x8, ctx.x_sinv, ctx.out_dtype, accumulate=True, out=old, amax_out=amax0)
            wgrad = wgrad.view(weight.shape)
            if model_state.use_fp8_ddp and not ctx.return_wgrad:
                # The FP8 DDP reducer quantises whole buckets with a cross-rank scale.
                wgrad.meta = wg_meta
            else:
                wgrad = _quantize_wgrad(wgrad, wg_meta, out=getattr(weight, '_grad_out', None))
            if ctx.return_wgrad:
                flat = wgrad.value.reshape(-1)
                pad = weight._flat_param._padded
                if pad:
                    flat = F.pad(flat, (0, pad))
                wgrad_ret = flat.view(torch.float32).view_as(weight._flat_param)
                wgrad_ret.meta = wg_meta
            else:
                weight.backward_grad_update(wgrad)
        ctx.x8 = ctx.w8 = None
        return dx, wgrad_ret, None, None, dbias


def _quantize_wgrad(wgrad, meta, out=None):
    """High-precision wgrad whose amax is already in ``meta.amax[0]`` → e4m3 ScalingTensor with an in-time scale.

    Without ``out`` the amax is MAX-reduced over the data-parallel group first so that all ranks share
    one scale and the bytes can be summed directly (the reference's rule).  With ``out`` – a slice of a
    sharded optimizer's flat symmetric gradient buffer – each rank keeps its own scale: the fused
    reduce kernel dequantises every rank's bytes with that rank's scale, so no collective runs here.
    """
    amax0 = meta.amax[0]
    if out is None and DistUtil.get_world_size(meta.group) > 1:
        dist.all_reduce(amax0, op=dist.ReduceOp.MAX, group=meta.group)
    value = _k.cast_to_fp8(wgrad, E4M3, meta.scale, scale_inv_out=meta.scale_inv, amax_in=amax0,
                           out=None if out is None else out.view(-1))
    return ScalingTensor(value.view(wgrad.shape), meta)


class FunctionalOverider:
    """Replaces ``F.linear`` by a version that routes ScalingTensor weights to the FP8 path."""
    EMPTY_GRAD_TENSOR = torch.nn.Parameter(torch.tensor([]))
    _holders = {}
    _installed = False

    @classmethod
    def override(cls):
        if cls._installed:
            return
        cls._installed = True
        F.linear = cls._get_wrapper_for_linear(F.linear)

    @classmethod
    def _holder(cls, dtype, device):
        """A zero-size leaf that requires grad, so backward runs even when the input needs no gradient."""
        key = (dtype, device)
        h = cls._holders.get(key)
        if h is None:
            h = torch.nn.Parameter(torch.empty(0, dtype=dtype, device=device))
            cls._holders[key] = h
        return h

    @classmethod
    def _get_wrapper_for_linear(cls, old_fn):
        def new_fn(input, weight, bias=None):
            """``linear(input, weight, bias=None)``; FP8 GEMM when ``weight`` is a ScalingTensor (or an FSDP FP8 flat view)."""
            if not isinstance(input, torch.Tensor):
                raise TypeError(f'input should be a torch.Tensor. current type: {type(input)}')
            if not isinstance(weight, (torch.Tensor, ScalingTensor)):
                raise TypeError(f'weight should be a torch.Tensor or ScalingTensor. current type: {type(weight)}')
            if bias is not None and not isinstance(bias, torch.Tensor):
                raise TypeError(f'bias should be a torch.Tensor. current type: {type(bias)}')
            if isinstance(weight, torch.Tensor) and not hasattr(weight, '_meta'):
                return old_fn(input, weight, bias=bias)
            if not hasattr(weight, '_scaling_metas'):
                raise ValueError('weight (ScalingTensor) should have _scaling_metas attribute.')
            model_state.ready_to_scale_tensor = True
            shape = input.shape
            if len(shape) != 2:
                input = input.reshape(-1, shape[-1])
            if torch.is_autocast_enabled(input.device.type):
                out_dtype = torch.get_autocast_dtype(input.device.type)
                input = input.to(out_dtype)
            else:
                out_dtype = input.dtype
            if out_dtype not in (torch.float32, torch.float16, torch.bfloat16):
                raise TypeError(f'unsupported activation dtype {out_dtype}')
            out = _FP8GemmFunction.apply(input, weight, weight._scaling_metas, cls._holder(out_dtype, input.device), bias)
            if len(shape) != 2:
                out = out.view(shape[:-1] + (-1, ))
            return out

        new_fn.__wrapped__ = old_fn
        return new_fn


FunctionalOverider.override()
