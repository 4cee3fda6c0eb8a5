"""Tensor / sequence-parallel FP8 linear.

``FP8LinearWithGradAccumulationAndAsyncCommunication`` has the call signature of the reference
(msamp/megatron/layers.py:30-221).  With sequence parallelism the activations entering the linear are
sharded along the token dimension over the tensor-parallel group; what the reference does with separate
NCCL calls around cuBLASLt, this implementation does inside fused kernels when the group shares an NVLink
domain (``msamp.parallel.fused``):

  forward   x_r --cast e4m3 (amax MAX-reduced over the TP group)--> shard in symmetric memory
            y = all-gather-rows(x8) · W8ᵀ                       one kernel (X18 + GEMM)
  backward  dx_r = reduce-scatter-rows(dy8 · W8)                one kernel (GEMM + X21)
            dW   = dy8ᵀ · all-gather-K(x8ᵀ)ᵀ                    one kernel (X19 + GEMM)

Without sequence parallelism dgrad is all-reduced over the TP group (asynchronously, overlapped with
the wgrad GEMM).  Anywhere the fused kernel cannot be used (CPU, one rank, shapes that are not tile
multiples) the unfused composition runs; it is also the test oracle.

Environment switches for simulated FP4 (same names as the reference): ``MSAMP_USE_WEIGHT_SIMULATE_FP4``,
``MSAMP_USE_WEIGHT_DIFFERENTIABLE_GRADIENT_ESTIMATOR``, ``MSAMP_USE_ACTIVATION_SIMULATE_FP4``.
"""
import os

import torch
import torch.distributed as dist

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingMeta, TypeCast
from msamp.megatron import parallel_state as mpu
from msamp.nn.functional import weight_fp8_pair
from msamp.nn.module import ScalingModule
from msamp.nn.parameter import ScalingParameter
from msamp.nn.state import model_state
from msamp.operators.fp4_quantize import FP4_QUANTIZER
from msamp.ops import cast as _k
from msamp.ops import gemm as _g
from msamp.parallel.fused import all_gather_cols, all_gather_rows, reduce_scatter_rows

E4M3, E5M2 = Dtypes.kfloat8_e4m3, Dtypes.kfloat8_e5m2

MSAMP_USE_WEIGHT_SIMULATE_FP4 = bool(int(os.getenv('MSAMP_USE_WEIGHT_SIMULATE_FP4', 0)))
MSAMP_USE_WEIGHT_DIFFERENTIABLE_GRADIENT_ESTIMATOR = bool(int(os.getenv('MSAMP_USE_WEIGHT_DIFFERENTIABLE_GRADIENT_ESTIMATOR', 0)))
MSAMP_USE_ACTIVATION_SIMULATE_FP4 = bool(int(os.getenv('MSAMP_USE_ACTIVATION_SIMULATE_FP4', 0)))


# False (or MSAMP_TP_FUSED=0) runs the NCCL collective + plain GEMM composition everywhere: the oracle of the fused kernels.
USE_FUSED_COLLECTIVES = bool(int(os.getenv('MSAMP_TP_FUSED', 1)))


def _fused_ctx(shard_bytes, out_bytes, device):
    if not USE_FUSED_COLLECTIVES or device.type != 'cuda' or mpu.get_tensor_model_parallel_world_size() == 1:
        return None
    ctx = mpu.get_fused_context(shard_bytes, out_bytes)
    return ctx if ctx.native else None


class FP8LinearWithGradAccumulationAndAsyncCommunication(torch.autograd.Function):
    """``y = x · Wᵀ + b`` for a tensor-parallel shard of W, with optional sequence-parallel gather / scatter."""
    @staticmethod
    def forward(ctx, input, weight, bias, gradient_accumulation_fusion, async_grad_allreduce, sequence_parallel):
        if gradient_accumulation_fusion:
            raise AssertionError('gradient_accumulation_fusion not supported for FP8LinearWithGradAccumulationAndAsyncCommunication')
        if sequence_parallel and async_grad_allreduce:
            raise AssertionError('sequence_parallel and async_grad_allreduce are mutually exclusive')
        tp_group = mpu.get_tensor_model_parallel_group()
        tp = mpu.get_tensor_model_parallel_world_size()
        metas = weight._scaling_metas
        in_meta = metas['input']
        out_dtype = input.dtype
        in_shape = input.shape
        x = input.contiguous().view(-1, in_shape[-1])
        if MSAMP_USE_ACTIVATION_SIMULATE_FP4:
            x = FP4_QUANTIZER.quantize_simulate_fp4_in_bf16(
                x.bfloat16(), format='e2m1', nan_existed=False, token_wise=True, outlier_clip=True, clip_threshold=0.99
            ).to(out_dtype)
        m_local, K = x.shape
        N = weight.shape[0]

        # quantise the local rows with a scale agreed over the TP group when they are a shard of one tensor
        saved_group, in_meta.group = in_meta.group, tp_group
        try:
            record = TypeCast._prepare_scale(x, in_meta, sync=bool(sequence_parallel) and tp > 1)
        finally:
            in_meta.group = saved_group
        amax_out = in_meta.amax[0] if record else None
        sinv_out = in_meta.scale_inv if record else None
        need_wgrad = weight.requires_grad and ctx.needs_input_grad[0] is not None
        x8, x8t = _k.cast_transpose_fp8(x, E4M3, in_meta.scale, amax_out, scale_inv_out=sinv_out)
        x_sinv = in_meta.scale_inv.clone()

        dge_scaled = None
        if MSAMP_USE_WEIGHT_SIMULATE_FP4:
            wq = FP4_QUANTIZER.quantize_simulate_fp4_in_bf16(
                weight.bfloat16(), format='e2m1', nan_existed=False, channel_wise=True,
                return_scaled_input_for_bwd=MSAMP_USE_WEIGHT_DIFFERENTIABLE_GRADIENT_ESTIMATOR
            )
            if MSAMP_USE_WEIGHT_DIFFERENTIABLE_GRADIENT_ESTIMATOR:
                wq, dge_scaled = wq
            w_st = wq.cast(E4M3)
            w8, w_sinv = w_st.value, w_st.meta.scale_inv
            w8t = _k.transpose_fp8(w8)
        else:
            w8, w8t, w_sinv = weight_fp8_pair(weight)

        fused = _fused_ctx(max(m_local * K, K * m_local), m_local * tp * max(N, K) * 2, x.device) if sequence_parallel and tp > 1 else None
        if sequence_parallel and tp > 1:
            if fused is not None and m_local % 128 == 0:
                view = fused.shard_view(m_local * K).view(m_local, K)
                view.copy_(x8)
                out = fused.ag_rows_gemm(view, E4M3, x_sinv, w8, E4M3, w_sinv, out_dtype, bias=bias if bias is None or bias.dtype == torch.float32 else None)
                if bias is not None and bias.dtype != torch.float32:
                    out.add_(bias)
            else:
                total = all_gather_rows(x8, tp_group)
                out = _g.gemm_fp8(total, E4M3, x_sinv, w8, E4M3, w_sinv, out_dtype, bias=bias)
            out_shape = (in_shape[0] * tp, ) + tuple(in_shape[1:-1]) + (N, )
        else:
            out = _g.gemm_fp8(x8, E4M3, x_sinv, w8, E4M3, w_sinv, out_dtype, bias=bias)
            out_shape = tuple(in_shape[:-1]) + (N, )

        ctx.metas, ctx.weight = metas, weight
        ctx.x8t, ctx.x_sinv, ctx.w8t, ctx.w_sinv = x8t, x_sinv, w8t, w_sinv
        ctx.use_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.async_grad_allreduce, ctx.sequence_parallel = async_grad_allreduce, sequence_parallel
        ctx.in_shape, ctx.out_dtype = in_shape, out_dtype
        ctx.dge_scaled = dge_scaled
        ctx.input_requires_grad = input.requires_grad
        ctx.m_local, ctx.K, ctx.N = m_local, K, N
        return out.view(out_shape)

    @staticmethod
    def backward(ctx, grad_output):
        tp_group = mpu.get_tensor_model_parallel_group()
        tp = mpu.get_tensor_model_parallel_world_size()
        metas, weight = ctx.metas, ctx.weight
        og_meta, wg_meta = metas['ograd'], metas['wgrad']
        dy = grad_output.contiguous().view(-1, grad_output.shape[-1])
        M_total, N = dy.shape
        K, m_local = ctx.K, ctx.m_local
        sp = ctx.sequence_parallel and tp > 1

        record = TypeCast._prepare_scale(dy, og_meta, sync=False)
        amax_out = og_meta.amax[0] if record else None
        sinv_out = og_meta.scale_inv if record else None
        dy8, dy8t = _k.cast_transpose_fp8(dy, E5M2, og_meta.scale, amax_out, scale_inv_out=sinv_out)
        dy_sinv = og_meta.scale_inv
        fused = _fused_ctx(max(m_local * K, K * m_local), M_total * max(N, K) * 2, dy.device) if sp else None

        handle = None
        if sp:
            if fused is not None and m_local % 128 == 0:
                dx = fused.gemm_rs(dy8, E5M2, dy_sinv, ctx.w8t, E4M3, ctx.w_sinv, ctx.out_dtype)
            else:
                full = _g.gemm_fp8(dy8, E5M2, dy_sinv, ctx.w8t, E4M3, ctx.w_sinv, ctx.out_dtype)
                dx = reduce_scatter_rows(full, tp_group)
        else:
            dx = _g.gemm_fp8(dy8, E5M2, dy_sinv, ctx.w8t, E4M3, ctx.w_sinv, ctx.out_dtype)
            if ctx.async_grad_allreduce and tp > 1:
                handle = dist.all_reduce(dx, group=tp_group, async_op=True)

        if weight.requires_grad:
            amax0 = wg_meta.amax[0]
            if sp:
                if fused is not None and m_local % 128 == 0:
                    rows_pad = (K + 255) // 256 * 256
                    view = fused.shard_view(rows_pad * m_local)[:K * m_local].view(K, m_local)
                    view.copy_(ctx.x8t)
                    wgrad = fused.ag_k_gemm(dy8t, E5M2, dy_sinv, view, E4M3, ctx.x_sinv, ctx.out_dtype, amax_out=amax0)
                else:
                    total_t = all_gather_cols(ctx.x8t, tp_group)
                    wgrad = _g.gemm_fp8(dy8t, E5M2, dy_sinv, total_t, E4M3, ctx.x_sinv, ctx.out_dtype, amax_out=amax0)
            else:
                wgrad = _g.gemm_fp8(dy8t, E5M2, dy_sinv, ctx.x8t, E4M3, ctx.x_sinv, ctx.out_dtype, amax_out=amax0)
            if ctx.dge_scaled is not None:
                wgrad.mul_(FP4_QUANTIZER.apply_DGE_item(ctx.dge_scaled).to(wgrad.dtype))
                _k.amax(wgrad, out=amax0)
            wgrad = wgrad.view(weight.shape)
            wgrad.meta = wg_meta    # consumers (FP8 local DDP, distributed optimizer) quantise / accumulate it
            weight.backward_grad_update(wgrad)
        grad_bias = dy.sum(0, dtype=torch.float32).to(ctx.bias_dtype) if ctx.use_bias else None
        if handle is not None:
            handle.wait()
        if sp:
            dx = dx.view((ctx.in_shape[0], ) + tuple(ctx.in_shape[1:]))
        else:
            dx = dx.view(ctx.in_shape)
        ctx.x8t = ctx.w8t = None
        return dx, None, grad_bias, None, None, None


def _new_fp8_weight(out_features, in_features, device, init_std, weight_qtype=Dtypes.kfloat16):
    w = torch.empty(out_features, in_features, device=device, dtype=torch.float32).normal_(0.0, init_std)
    meta = ScalingMeta(weight_qtype, window_size=1, device=w.device)
    return ScalingParameter(w.cast(weight_qtype, meta=meta))


class _ParallelLinearBase(ScalingModule):
    DEFAULT_WINDOW_SIZE = 16

    def _make_metas(self, device):
        self.scaling_metas = dict(
            input=ScalingMeta(E4M3, window_size=self.DEFAULT_WINDOW_SIZE, device=device),
            wgrad=ScalingMeta(E4M3, window_size=1, device=device),
            ograd=ScalingMeta(E5M2, window_size=self.DEFAULT_WINDOW_SIZE, device=device),
        )
        self.weight._scaling_metas = self.scaling_metas
        model_state.register_scaling_metas(self, None)


class ColumnParallelLinear(_ParallelLinearBase):
    """``Y = X Wᵀ + b`` with the output features split over the tensor-parallel group (W shard ``[out/tp, in]``).

    With ``sequence_parallel`` the input arrives sharded along dim 0 and is gathered inside the GEMM kernel.
    """
    def __init__(self, in_features, out_features, bias=True, sequence_parallel=False, init_std=0.02, device=None, gather_output=False):
        super().__init__()
        tp = mpu.get_tensor_model_parallel_world_size()
        if out_features % tp:
            raise ValueError('out_features must be divisible by the tensor-parallel size')
        self.in_features, self.out_features, self.sequence_parallel, self.gather_output = in_features, out_features, sequence_parallel, gather_output
        dev = torch.device(device) if device is not None else torch.device('cpu')
        self.weight = _new_fp8_weight(out_features // tp, in_features, dev, init_std)
        self.weight.tensor_model_parallel = True
        self.bias = torch.nn.Parameter(torch.zeros(out_features // tp, device=dev)) if bias else None
        if self.bias is not None:
            self.bias.tensor_model_parallel = True    # a shard, not a replica: counts on every rank in gradient norms
        self._make_metas(dev)

    def forward(self, x):
        tp = mpu.get_tensor_model_parallel_world_size()
        out = FP8LinearWithGradAccumulationAndAsyncCommunication.apply(
            x, self.weight, self.bias, False, (not self.sequence_parallel) and tp > 1, self.sequence_parallel
        )
        if self.gather_output and tp > 1:
            parts = [torch.empty_like(out) for _ in range(tp)]
            dist.all_gather(parts, out.contiguous(), group=mpu.get_tensor_model_parallel_group())
            out = torch.cat(parts, -1)
        return out


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return reduce_scatter_rows(x.contiguous().view(-1, x.shape[-1]), mpu.get_tensor_model_parallel_group()).view(
            (x.shape[0] // mpu.get_tensor_model_parallel_world_size(), ) + tuple(x.shape[1:])
        )

    @staticmethod
    def backward(ctx, g):
        tp_group = mpu.get_tensor_model_parallel_group()
        return all_gather_rows(g.contiguous().view(-1, g.shape[-1]), tp_group).view((g.shape[0] * dist.get_world_size(tp_group), ) + tuple(g.shape[1:]))


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        dist.all_reduce(x, group=mpu.get_tensor_model_parallel_group())
        return x

    @staticmethod
    def backward(ctx, g):
        return g


class _RowParallelFn(torch.autograd.Function):
    """Row-parallel linear with the reduce-scatter (forward) and the all-gather (backward) inside the GEMM kernels."""
    @staticmethod
    def forward(ctx, input, weight, dummy):
        tp_group = mpu.get_tensor_model_parallel_group()
        tp = mpu.get_tensor_model_parallel_world_size()
        metas = weight._scaling_metas
        in_meta = metas['input']
        x = input.contiguous().view(-1, input.shape[-1])
        M, K_local = x.shape
        N = weight.shape[0]
        record = TypeCast._prepare_scale(x, in_meta, sync=False)
        x8, x8t = _k.cast_transpose_fp8(x, E4M3, in_meta.scale, in_meta.amax[0] if record else None,
                                        scale_inv_out=in_meta.scale_inv if record else None)
        x_sinv = in_meta.scale_inv.clone()
        w8, w8t, w_sinv = weight_fp8_pair(weight)
        fused = _fused_ctx((M // tp) * max(N, K_local), M * N * 2, x.device)
        if fused is not None and (M // tp) % 128 == 0:
            out = fused.gemm_rs(x8, E4M3, x_sinv, w8, E4M3, w_sinv, input.dtype)
        else:
            out = reduce_scatter_rows(_g.gemm_fp8(x8, E4M3, x_sinv, w8, E4M3, w_sinv, input.dtype), tp_group)
        ctx.metas, ctx.weight = metas, weight
        ctx.x8t, ctx.x_sinv, ctx.w8t, ctx.w_sinv = x8t, x_sinv, w8t, w_sinv
        ctx.in_shape, ctx.out_dtype, ctx.M, ctx.N, ctx.K = input.shape, input.dtype, M, N, K_local
        return out.view((input.shape[0] // tp, ) + tuple(input.shape[1:-1]) + (N, ))

    @staticmethod
    def backward(ctx, grad_output):
        tp_group = mpu.get_tensor_model_parallel_group()
        tp = mpu.get_tensor_model_parallel_world_size()
        metas, weight = ctx.metas, ctx.weight
        og_meta, wg_meta = metas['ograd'], metas['wgrad']
        dy = grad_output.contiguous().view(-1, grad_output.shape[-1])    # [M/tp, N], a row shard
        m_local, N = dy.shape
        saved, og_meta.group = og_meta.group, tp_group
        try:
            record = TypeCast._prepare_scale(dy, og_meta, sync=tp > 1)
        finally:
            og_meta.group = saved
        dy8, dy8t = _k.cast_transpose_fp8(dy, E5M2, og_meta.scale, og_meta.amax[0] if record else None,
                                          scale_inv_out=og_meta.scale_inv if record else None)
        dy_sinv = og_meta.scale_inv
        fused = _fused_ctx(m_local * max(N, ctx.K), ctx.M * N * 2, dy.device)
        use_fused = fused is not None and m_local % 128 == 0
        # dgrad: dx[M, K] = all-gather-rows(dy8) · (W8ᵀ)ᵀ
        if use_fused:
            view = fused.shard_view(m_local * N).view(m_local, N)
            view.copy_(dy8)
            dx = fused.ag_rows_gemm(view, E5M2, dy_sinv, ctx.w8t, E4M3, ctx.w_sinv, ctx.out_dtype)
        else:
            dx = _g.gemm_fp8(all_gather_rows(dy8, tp_group), E5M2, dy_sinv, ctx.w8t, E4M3, ctx.w_sinv, ctx.out_dtype)
        if weight.requires_grad:
            amax0 = wg_meta.amax[0]
            # wgrad: dW[N, K] = all-gather-K(dy8ᵀ) · (x8ᵀ)ᵀ  ==  (x8ᵀ · all-gather-K(dy8ᵀ)ᵀ)ᵀ ; computed as D'[K, N] then transposed view
            if use_fused:
                rows_pad = (N + 255) // 256 * 256
                view = fused.shard_view(rows_pad * m_local)[:N * m_local].view(N, m_local)
                view.copy_(dy8t)
                wgrad_t = fused.ag_k_gemm(ctx.x8t, E4M3, ctx.x_sinv, view, E5M2, dy_sinv, ctx.out_dtype, amax_out=amax0)
            else:
                wgrad_t = _g.gemm_fp8(ctx.x8t, E4M3, ctx.x_sinv, all_gather_cols(dy8t, tp_group), E5M2, dy_sinv, ctx.out_dtype, amax_out=amax0)
            wgrad = wgrad_t.t().contiguous().view(weight.shape)
            wgrad.meta = wg_meta
            weight.backward_grad_update(wgrad)
        ctx.x8t = ctx.w8t = None
        return dx.view(ctx.in_shape), None, None


class RowParallelLinear(_ParallelLinearBase):
    """``Y = X Wᵀ + b`` with the input features split over the tensor-parallel group (W shard ``[out, in/tp]``).

    The partial products are summed over the group: reduce-scattered along dim 0 with ``sequence_parallel``
    (inside the GEMM kernel when possible), all-reduced otherwise.  The bias is added after the reduction.
    """
    def __init__(self, in_features, out_features, bias=True, sequence_parallel=False, init_std=0.02, device=None):
        super().__init__()
        tp = mpu.get_tensor_model_parallel_world_size()
        if in_features % tp:
            raise ValueError('in_features must be divisible by the tensor-parallel size')
        self.in_features, self.out_features, self.sequence_parallel = in_features, out_features, sequence_parallel
        dev = torch.device(device) if device is not None else torch.device('cpu')
        self.weight = _new_fp8_weight(out_features, in_features // tp, dev, init_std)
        self.weight.tensor_model_parallel = True
        self.bias = torch.nn.Parameter(torch.zeros(out_features, device=dev)) if bias else None
        self._holder = torch.nn.Parameter(torch.empty(0, device=dev))
        self._make_metas(dev)

    def forward(self, x):
        tp = mpu.get_tensor_model_parallel_world_size()
        if self.sequence_parallel and tp > 1:
            out = _RowParallelFn.apply(x, self.weight, self._holder)
        else:
            out = FP8LinearWithGradAccumulationAndAsyncCommunication.apply(x, self.weight, None, False, False, False)
            if tp > 1:
                out = _AllReduce.apply(out)
        if self.bias is not None:
            out = out + self.bias.to(out.dtype)
        return out
