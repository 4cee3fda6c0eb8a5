"""Full-shard (ZeRO-3) data parallelism for FP8 linears, built on the fused gather-GEMM kernels.

Every FP8Linear weight ``W [N, K]`` is split by rows over the data-parallel group; a rank permanently holds
only its e4m3 shard ``W_r [N/W, K]`` (and the shard's transpose), its scaled-fp16 master shard and its Adam
moment shards.  One scale per *tensor* is kept consistent by MAX-reducing the amax over the shards before
every re-quantisation (the reference's rule, msamp/optim/adamw.py:306-337).  The e4m3 shards live permanently in
symmetric (peer-mapped) memory, so the gather kernels read them where they are; everything that is not a sharded
linear (embeddings, LayerNorms, biases) is sharded ZeRO-style by ``msamp.parallel.hp_shard.HighPrecisionShards``.

  forward   y  = x8 · all-gather-rows(W8_r)ᵀ           parameter all-gather fused into the GEMM
  backward  dx = dy8 · all-gather-K(W8ᵀ_r)ᵀ            parameter all-gather (transposed shards) fused into the GEMM
            dW_r = reduce-scatter-rows(dy8ᵀ · x8)      gradient reduce-scatter fused into the GEMM; the owner keeps its rows

The reference routes FP8 bytes through torch's FSDP by patching its private flat-parameter handle and
all-reduces full gradients before slicing (msamp/fsdp/fully_sharded_data_parallel.py:14-63); torch's
private FSDP API has since moved, so this module owns the sharding itself.  ``FsdpReplacer`` plus
``msamp.optim.FSDPAdamW`` remain available for use with torch FSDP (``use_orig_params=True``).
"""
import torch
import torch.distributed as dist

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingMeta, ScalingTensor, TypeCast
from msamp.common.utils.dist import DistUtil
from msamp.nn.linear import FP8Linear
from msamp.nn.module import ScalingModule
from msamp.nn.parameter import ScalingParameter
from msamp.nn.state import model_state
from msamp.ops import cast as _k
from msamp.ops import gemm as _g
from msamp.parallel.fused import FusedGemmContext, all_gather_cols, all_gather_rows, reduce_scatter_rows

E4M3, E5M2, F16 = Dtypes.kfloat8_e4m3, Dtypes.kfloat8_e5m2, Dtypes.kfloat16


class _ShardedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, module, holder, bias):
        fs = module._fsdp
        in_meta = module.scaling_metas['input']
        x2 = x.contiguous().view(-1, x.shape[-1])
        record = TypeCast._prepare_scale(x2, in_meta, sync=False)
        x8, x8t = _k.cast_transpose_fp8(x2, E4M3, in_meta.scale, in_meta.amax[0] if record else None,
                                        scale_inv_out=in_meta.scale_inv if record else None)
        x_sinv = in_meta.scale_inv.clone()
        w8, w_sinv = module.weight_shard, module.weight_meta.scale_inv
        rows, K = w8.shape
        fused = fs.ctx if (fs.ctx is not None and fs.ctx.native and rows % 128 == 0 and module.resident) else None
        if fused is not None:
            fs.fused_calls += 1
            out = fused.ag_rows_gemm(w8, E4M3, w_sinv, x8, E4M3, x_sinv, x.dtype, bias=bias if bias is None or bias.dtype == torch.float32 else None,
                                     shard_is='b')
            if bias is not None and bias.dtype != torch.float32:
                out.add_(bias)
        else:
            fs.unfused_calls += 1
            out = _g.gemm_fp8(x8, E4M3, x_sinv, all_gather_rows(w8, fs.group), E4M3, w_sinv, x.dtype, bias=bias)
        ctx.module, ctx.x8t, ctx.x_sinv = module, x8t, x_sinv
        ctx.in_shape, ctx.out_dtype = x.shape, x.dtype
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.input_requires_grad = x.requires_grad
        return out.view(tuple(x.shape[:-1]) + (out.shape[-1], ))

    @staticmethod
    def backward(ctx, grad_output):
        module = ctx.module
        fs = module._fsdp
        og_meta, wg_meta = module.scaling_metas['ograd'], module.scaling_metas['wgrad']
        dy = grad_output.contiguous().view(-1, grad_output.shape[-1])
        T, N = dy.shape
        record = TypeCast._prepare_scale(dy, og_meta, sync=False)
        dy8, dy8t = _k.cast_transpose_fp8(dy, E5M2, og_meta.scale, og_meta.amax[0] if record else None,
                                          scale_inv_out=og_meta.scale_inv if record else None)
        dy_sinv = og_meta.scale_inv
        w8t, w_sinv = module.weight_shard_t, module.weight_meta.scale_inv    # [K, N/W]
        K, n_local = w8t.shape
        fused_ok = fs.ctx is not None and fs.ctx.native and module.resident
        dx = None
        if ctx.input_requires_grad:
            if fused_ok and n_local % 128 == 0:
                fs.fused_calls += 1
                dx = fs.ctx.ag_k_gemm(dy8, E5M2, dy_sinv, w8t, E4M3, w_sinv, ctx.out_dtype)    # the resident transposed shard, no copy
            else:
                fs.unfused_calls += 1
                dx = _g.gemm_fp8(dy8, E5M2, dy_sinv, all_gather_cols(w8t, fs.group), E4M3, w_sinv, ctx.out_dtype)
            dx = dx.view(ctx.in_shape)
        # weight gradient of the local batch, reduced over ranks; this rank keeps the rows of its shard.  The partial
        # products cross NVLink as bf16 (half the bytes of fp32; every rank's partial is rounded once before the fp32 sum).
        if fused_ok and n_local % 128 == 0:
            fs.fused_calls += 1
            part = fs.ctx.gemm_rs(dy8t, E5M2, dy_sinv, ctx.x8t, E4M3, ctx.x_sinv, torch.bfloat16).float()
        else:
            fs.unfused_calls += 1
            full = _g.gemm_fp8(dy8t, E5M2, dy_sinv, ctx.x8t, E4M3, ctx.x_sinv, torch.float32)
            part = reduce_scatter_rows(full, fs.group)
        part.div_(fs.world)
        # quantise with a scale agreed over the shards of this tensor
        amax0 = wg_meta.amax[0]
        _k.amax(part, out=amax0)
        if fs.world > 1:
            dist.all_reduce(amax0, op=dist.ReduceOp.MAX, group=fs.group)
        old = module.master.grad
        if old is not None:
            part.add_(old.float())
            _k.amax(part, out=amax0)
            if fs.world > 1:
                dist.all_reduce(amax0, op=dist.ReduceOp.MAX, group=fs.group)
        value = _k.cast_to_fp8(part, E4M3, wg_meta.scale, scale_inv_out=wg_meta.scale_inv, amax_in=amax0)
        module.master.grad = ScalingTensor(value, wg_meta)
        dbias = dy.sum(0, dtype=torch.float32).to(ctx.bias_dtype) if ctx.has_bias else None
        ctx.x8t = None
        return dx, None, None, dbias


class ShardedFP8Linear(ScalingModule):
    """A linear layer whose FP8 weight, master weight and optimizer state are split by rows over the group."""
    def __init__(self, linear, fsdp):
        super().__init__()
        self._fsdp = fsdp
        self.in_features, self.out_features = linear.in_features, linear.out_features
        W, r = fsdp.world, fsdp.rank
        if self.out_features % W:
            raise ValueError(f'out_features={self.out_features} is not divisible by the shard count {W}')
        rows = self.out_features // W
        w = linear.weight
        full = w.float() if isinstance(w, ScalingTensor) else w.detach().float()
        dev = full.device
        shard = full[r * rows:(r + 1) * rows].contiguous()
        # one scale for the whole tensor
        amax = full.abs().max()
        self.master = ScalingParameter(shard.cast(F16, meta=_meta_from_amax(F16, amax, dev)))
        self.weight_meta = _meta_from_amax(E4M3, amax, dev)
        self.weight_shard = _k.cast_to_fp8(shard, E4M3, self.weight_meta.scale)
        self.weight_shard_t = _k.transpose_fp8(self.weight_shard)
        self.resident = False    # True once both copies live in the fused context's symmetric buffer
        self.bias = linear.bias
        self.scaling_metas = linear.scaling_metas if isinstance(linear, FP8Linear) else dict(
            input=ScalingMeta(E4M3, window_size=FP8Linear.DEFAULT_WINDOW_SIZE, device=dev),
            wgrad=ScalingMeta(E4M3, window_size=1, device=dev),
            ograd=ScalingMeta(E5M2, window_size=FP8Linear.DEFAULT_WINDOW_SIZE, device=dev),
        )
        self.master._scaling_metas = self.scaling_metas
        self._holder = torch.nn.Parameter(torch.empty(0, device=dev))

    def resident_bytes(self):
        """Symmetric memory both FP8 copies need: the shard, and its transpose with the row count rounded up to the
        256-row tile of the K-gather kernel (whole tiles are copied between ranks)."""
        rows, K = self.weight_shard.shape
        pad_k = (K + 255) // 256 * 256
        return ((rows * K + 1023) // 1024 + (pad_k * rows + 1023) // 1024 + 2) * 1024

    def make_resident(self, ctx):
        """Move the FP8 shard and its transpose into ``ctx``'s symmetric buffer (every rank in the same order)."""
        rows, K = self.weight_shard.shape
        pad_k = (K + 255) // 256 * 256
        w = ctx.resident_view(rows * K).view(rows, K)
        wt = ctx.resident_view(pad_k * rows)[:K * rows].view(K, rows)
        w.copy_(self.weight_shard)
        wt.copy_(self.weight_shard_t)
        self.weight_shard, self.weight_shard_t = w, wt
        self.resident = True

    def forward(self, x):
        model_state.ready_to_scale_tensor = True
        return _ShardedLinearFn.apply(x, self, self._holder, self.bias)

    @torch.no_grad()
    def requantize(self):
        """Master shard → e4m3 shard (and its transpose) with the tensor-wide scale."""
        fs = self._fsdp
        amax = self.weight_meta.amax[0]
        amax.copy_(self.master.meta.amax[0])
        if fs.world > 1:
            dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=fs.group)
        self.weight_meta.reset_scaling_factor()
        torch.reciprocal(self.weight_meta.scale, out=self.weight_meta.scale_inv)
        factor = self.weight_meta.scale * self.master.meta.scale_inv
        # in place: the shards keep their addresses (peers hold mappings of them).  No peer reads them between the last
        # fused call of backward and the first of the next forward: every fused call ends with a cross-rank barrier.
        _k.cast_to_fp8(self.master.value, E4M3, factor, out=self.weight_shard.view(-1))
        _k.transpose_fp8(self.weight_shard, out=self.weight_shard_t)

    def extra_repr(self):
        return f'in_features={self.in_features}, out_features={self.out_features}, shards={self._fsdp.world}'


def _meta_from_amax(qtype, amax, device):
    meta = ScalingMeta(qtype, window_size=1, device=device)
    meta.amax[0] = amax
    meta.reset_scaling_factor()
    torch.reciprocal(meta.scale, out=meta.scale_inv)
    meta.amax_counter += 1    # keep the given scale when casting with this meta
    return meta


class FP8FullyShardedDataParallel(torch.nn.Module):
    """Wrap ``module``: shard every (FP8)Linear over ``process_group``, replicate and all-reduce everything else.

    Use ``optimizer = fsdp.build_optimizer(torch.optim.AdamW, lr=...)`` (low-bit Adam on the master shards and on
    the replicated high-precision parameters) and call ``fsdp.step(optimizer)`` after ``backward``.
    """
    def __init__(self, module, process_group=None, min_shard_numel=0, **unused):
        super().__init__()
        self.group = process_group
        self.world = DistUtil.get_world_size(process_group)
        self.rank = DistUtil.get_rank(process_group)
        self.ctx = None
        self.sharded = []
        self.fused_calls = self.unfused_calls = 0    # GEMMs of sharded linears that took / did not take the fused kernels
        biggest_shard, biggest_out, resident = 0, 0, 0
        module = self._convert(module, min_shard_numel)
        for m in self.sharded:
            rows, K = m.weight_shard.shape
            pad_k = (K + 255) // 256 * 256
            biggest_shard = max(biggest_shard, rows * K, pad_k * rows)
            biggest_out = max(biggest_out, m.out_features * K * 2)    # bf16 partial products
            resident += m.resident_bytes()
        first = self.sharded[0].weight_shard if self.sharded else None
        if first is not None and first.is_cuda and self.world > 1:
            self.ctx = FusedGemmContext(process_group, biggest_shard, biggest_out, resident_bytes=resident)
            if self.ctx.native:
                for m in self.sharded:
                    m.make_resident(self.ctx)
        self.module = module
        model_state.register_scaling_metas(module, None)
        self.hp_params = [p for p in module.parameters() if not isinstance(p, ScalingParameter) and p.numel() > 0]
        if self.world > 1:
            src = dist.get_global_rank(process_group, 0) if process_group is not None else 0
            for p in self.hp_params:
                dist.broadcast(p.data, src=src, group=process_group)
        from msamp.parallel.hp_shard import HighPrecisionShards
        dev = first.device if first is not None else (self.hp_params[0].device if self.hp_params else torch.device('cpu'))
        self.hp = HighPrecisionShards(self.hp_params, process_group, shard=True, device=dev)
        self._flatten_weight_metas(dev)

    def _flatten_weight_metas(self, dev):
        """Put the scalars that the re-quantisation of the weight shards reads and writes (the masters' amax and scale_inv,
        the shards' amax, scale and scale_inv) into flat vectors, each meta keeping a view: one MAX all-reduce, one
        vectorised scale computation and one multi-tensor cast then serve all sharded linears of a step."""
        n = len(self.sharded)
        if n == 0:
            return
        f = lambda fill: torch.full((n, ), fill, dtype=torch.float32, device=dev)    # noqa: E731
        self._m_amax, self._m_sinv = f(0.0), f(1.0)
        self._w_amax, self._w_scale, self._w_sinv, self._factor = f(0.0), f(1.0), f(1.0), f(1.0)
        for i, m in enumerate(self.sharded):
            for meta, amax, scale, sinv in ((m.master.meta, self._m_amax, None, self._m_sinv), (m.weight_meta, self._w_amax, self._w_scale, self._w_sinv)):
                was_locked, meta.locked = meta.locked, False
                amax[i:i + 1].copy_(meta.amax[0:1])
                meta.amax = amax[i:i + 1]
                sinv[i].copy_(meta.scale_inv)
                meta.scale_inv = sinv[i:i + 1].view(())
                if scale is not None:
                    scale[i].copy_(meta.scale)
                    meta.scale = scale[i:i + 1].view(())
                meta.locked = was_locked
        self._factor_views = [self._factor[i:i + 1].view(()) for i in range(n)]

    @torch.no_grad()
    def _requantize_all(self):
        """Master shards -> e4m3 shards (and their transposes), every tensor with its tensor-wide scale: the amax of
        every master is agreed across the shards by ONE MAX all-reduce, the scales come from one vectorised application of
        the power-of-two rule, and one multi-tensor launch casts all shards (``ShardedFP8Linear.requantize`` is the
        per-module form of the same arithmetic)."""
        ms = self.sharded
        if not ms:
            return
        from msamp.common.dtype import Floating
        from msamp.ops import multi_tensor as _mt
        self._w_amax.copy_(self._m_amax)
        if self.world > 1:
            dist.all_reduce(self._w_amax, op=dist.ReduceOp.MAX, group=self.group)
        self._w_scale.copy_(ScalingMeta.compute_scaling_factor(self._w_amax, self._w_scale, Floating.qfp_max[E4M3], 0))
        torch.reciprocal(self._w_scale, out=self._w_sinv)
        torch.mul(self._w_scale, self._m_sinv, out=self._factor)
        # in place: the shards keep their addresses (peers hold mappings of them).  No peer reads them between the last
        # fused call of backward and the first of the next forward: every fused call ends with a cross-rank barrier.
        _mt.cast_to_fp8_multi([m.master.value.view(-1) for m in ms], [m.weight_shard.view(-1) for m in ms], E4M3, self._factor_views,
                              tag='fsdp_requant')
        for m in ms:
            _k.transpose_fp8(m.weight_shard, out=m.weight_shard_t)

    def _convert(self, module, min_numel):
        if isinstance(module, (torch.nn.Linear, FP8Linear)) and not getattr(module, 'use_fp32_linear', False):
            if module.in_features * module.out_features >= min_numel and module.out_features % self.world == 0:
                sharded = ShardedFP8Linear(module, self)
                self.sharded.append(sharded)
                return sharded
            return module
        for name, child in list(module.named_children()):
            setattr(module, name, self._convert(child, min_numel))
        return module

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def master_parameters(self):
        """Parameters an optimizer should update: master shards of the sharded linears + the high-precision parameters this rank owns."""
        return [m.master for m in self.sharded] + self.hp.owned()

    def build_optimizer(self, torch_cls=torch.optim.AdamW, **kwargs):
        from msamp.optim import LBAdam, LBAdamW
        cls = LBAdamW if torch_cls is torch.optim.AdamW else LBAdam
        return cls(self.master_parameters(), exp_avg_dtype=torch.uint8, exp_avg_sq_dtype=torch.float16, **kwargs)

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm):
        """Global-norm clipping.  Every gradient is held by exactly one rank here (shards of the linears, owners of the
        other parameters), so the squared norms are summed over the group.  Call after ``hp.reduce_grads()`` (``step``
        does both in the right order when given ``clip_grad``)."""
        from msamp.ops import multi_tensor as _mt
        grads = [m.master.grad for m in self.sharded if m.master.grad is not None]
        grads += [p.grad for p in self.hp.owned() if p.grad is not None]
        dev = self.sharded[0].master.device if self.sharded else self.hp_params[0].device
        stats = _mt.grad_sumsq(grads, out=torch.zeros(2, dtype=torch.float32, device=dev), tag='fsdp_norm')
        if self.world > 1:
            dist.all_reduce(stats, group=self.group)
        _mt.clip_by_sumsq(grads, stats[0:1], max_norm, tag='fsdp_clip')
        return stats[0].sqrt()

    @torch.no_grad()
    def step(self, optimizer, clip_grad=0.0):
        """Reduce the high-precision gradients to their owners, (clip,) update, publish the owners' parameters,
        re-quantise the weight shards, clear gradients."""
        self.hp.reduce_grads()
        if clip_grad > 0:
            self.clip_grad_norm_(clip_grad)
        optimizer.step()
        self.hp.gather_params()
        self._requantize_all()
        for m in self.sharded:
            m.master.grad = None
        self.hp.clear_grads()

    def close(self):
        """Release the symmetric buffers of the fused kernels (collective over the group, after the last step)."""
        if self.ctx is not None:
            if self.ctx.native:
                torch.cuda.synchronize()
                for m in self.sharded:    # resident shards alias the symmetric buffer: keep the values in ordinary memory
                    if getattr(m, 'resident', False):
                        m.weight_shard, m.weight_shard_t = m.weight_shard.clone(), m.weight_shard_t.clone()
                        m.resident = False
                torch.cuda.synchronize()
            self.ctx.close()
            self.ctx = None

    def memory_per_rank(self):
        """Bytes of persistent parameter/optimizer storage on this rank for the sharded layers (fp8 W, W^T, fp16 master)."""
        return sum(m.weight_shard.numel() * 2 + m.master.numel() * 2 for m in self.sharded)


__all__ = ['FP8FullyShardedDataParallel', 'ShardedFP8Linear']
