"""FP8 DistributedDataParallel.

A drop-in subclass of torch's DDP.  High-precision parameters go through torch's own reducer;
FP8Linear weights (DDP-ignored ScalingParameters) are handled by ``_ScalingTensorReducer``: they are
packed in reverse registration order into byte-capped buckets, and when the last gradient of a bucket
arrives the bucket's amax values are MAX-reduced, a common scale is derived (pre-scaled by 1/sqrt(W)
against overflow of the sum), the gradients are quantised to e4m3 into one flat buffer, and the buffer
is SUM-reduced as FP8 numbers asynchronously; ``scale_inv`` is divided by W so the result is the mean.
``_DDPSink`` resets the bucket bookkeeping in forward and waits for the collectives at the end of backward.
(reference: msamp/nn/distributed.py:18-264)

For the sharded / fused NVLink path see ``msamp.parallel.ZeroShardedOptimizer``.
"""
import math

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as _TorchDDP

from msamp.common.dtype import Dtypes, Floating
from msamp.common.tensor import ScalingMeta, ScalingTensor
from msamp.nn.parameter import ScalingParameter
from msamp.nn.state import model_state
from msamp.operators.dist_op import DistOp
from msamp.ops import cast as _k

E4M3 = Dtypes.kfloat8_e4m3


class _ScalingTensorReducer:
    """Bucketed FP8 all-reduce of ScalingTensor gradients."""
    def __init__(self, parameters, process_group, bucket_bytes_cap):
        parameters = list(parameters)
        if not all(isinstance(p, ScalingTensor) for p in parameters):
            raise ValueError('All parameters must be ScalingTensor')
        if parameters and not all(p.device == parameters[0].device for p in parameters):
            raise ValueError('All parameters must be on the same device')
        self.parameters = parameters
        self.device = parameters[0].device if parameters else torch.device('cpu')
        self.process_group = process_group
        self.bucket_bytes_cap = bucket_bytes_cap
        self.param_to_id = {id(p): i for i, p in enumerate(parameters)}
        self.buffer = None
        self.dist_handles = []
        self.sync = True    # False while the owning DDP module is inside no_sync()
        self.bucket_unreduced_param_ids = {}
        self.reduction_stream = torch.cuda.Stream(device=self.device) if self.device.type == 'cuda' else None
        self._build_buckets()
        for p in parameters:
            p.register_backward_post_hook(self._make_hook(p))

    def _build_buckets(self):
        self.param_id_to_bucket_id, self.bucket_to_param_ids, self.bucket_to_range = {}, {}, {}
        nbytes, bucket, start = 0, 0, 0
        for p in reversed(self.parameters):
            pid = self.param_to_id[id(p)]
            self.param_id_to_bucket_id[pid] = bucket
            self.bucket_to_param_ids.setdefault(bucket, []).append(pid)
            nbytes += p.numel()
            if nbytes >= self.bucket_bytes_cap:
                self.bucket_to_range[bucket] = (start, start + nbytes)
                start += nbytes
                bucket += 1
                nbytes = 0
        if nbytes > 0:
            self.bucket_to_range[bucket] = (start, start + nbytes)

    def reset_buckets(self):
        if self.bucket_unreduced_param_ids:
            raise RuntimeError(f'some gradients not reduced: {list(self.bucket_unreduced_param_ids.keys())}')
        self.bucket_unreduced_param_ids = {k: set(v) for k, v in self.bucket_to_param_ids.items()}

    def wait(self):
        for h in self.dist_handles:
            if h is not None:
                h.wait()
        self.dist_handles.clear()
        if self.reduction_stream is not None:
            torch.cuda.current_stream().wait_stream(self.reduction_stream)

    def _make_hook(self, param):
        pid = self.param_to_id[id(param)]
        bucket = self.param_id_to_bucket_id[pid]

        def hook(*args, **kwargs):
            pending = self.bucket_unreduced_param_ids.get(bucket)
            if pending is None or pid not in pending:
                raise RuntimeError('gradient is already reduced')
            pending.remove(pid)
            if not pending:
                if self.sync:
                    self._reduce_bucket(bucket)
                # inside DDP.no_sync() the high-precision gradients stay as they are and keep accumulating; the
                # backward pass that synchronises quantises and reduces their sum (the reference reduces every time)
                self.bucket_unreduced_param_ids.pop(bucket)

        return hook

    def _reduce_bucket(self, bucket):
        world = dist.get_world_size(self.process_group)
        params = [self.parameters[pid] for pid in self.bucket_to_param_ids[bucket]]
        grads = [p.grad for p in params]
        if self.buffer is None:
            self.buffer = torch.empty(sum(p.numel() for p in self.parameters), dtype=torch.uint8, device=self.device)
        lo, hi = self.bucket_to_range[bucket]
        flat = self.buffer[lo:hi]
        stream_ctx = torch.cuda.stream(self.reduction_stream) if self.reduction_stream is not None else _NullCtx()
        if self.reduction_stream is not None:
            self.reduction_stream.wait_stream(torch.cuda.current_stream())
        with stream_ctx:
            metas = []
            amaxs = []
            for g in grads:
                if isinstance(g, ScalingTensor):
                    raise RuntimeError('FP8 DDP expects high-precision gradients carrying a .meta (set model_state.use_fp8_ddp)')
                meta = getattr(g, 'meta', None) or ScalingMeta(E4M3, device=g.device)
                metas.append(meta)
                amaxs.append(_k.amax(g))
            amax = torch.stack(amaxs)
            dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.process_group)
            ones = torch.ones_like(amax)
            scales = ScalingMeta.compute_scaling_factor(amax, ones, Floating.qfp_max[E4M3], 0) * (1.0 / math.sqrt(world))
            off = 0
            for i, (p, g, meta) in enumerate(zip(params, grads, metas)):
                meta.amax[0] = amax[i]
                meta.scale.copy_(scales[i])
                n = g.numel()
                view = flat[off:off + n]
                _k.cast_to_fp8(g.contiguous(), E4M3, meta.scale, scale_inv_out=meta.scale_inv, out=view)
                q = ScalingTensor(view.view(g.shape), meta)
                q.div_(world)
                p.grad = q
                off += n
        if self.reduction_stream is not None:
            torch.cuda.current_stream().wait_stream(self.reduction_stream)
        self.dist_handles.append(DistOp.all_reduce(flat, E4M3, dist.ReduceOp.SUM, group=self.process_group, async_op=True))


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class _DDPSink(torch.autograd.Function):
    """Identity on the inputs; marks the start of a forward pass and the end of the matching backward pass."""
    @staticmethod
    def forward(ctx, reducer, anchor, *inputs):
        ctx.reducer = reducer
        ctx.set_materialize_grads(False)
        reducer.reset_buckets()
        return inputs

    @staticmethod
    def backward(ctx, *grads):
        ctx.reducer.wait()
        return (None, None) + grads


class FP8DistributedDataParallel(_TorchDDP):
    """``torch.nn.parallel.DistributedDataParallel`` that also reduces FP8Linear weight gradients in FP8."""
    def __init__(self, module, *args, **kwargs):
        super().__init__(module, *args, **kwargs)
        scaling = [p for p in self.module.parameters() if isinstance(p, ScalingParameter)]
        self.scaling_tensor_reducer = None
        if scaling:
            cap = getattr(self, 'bucket_bytes_cap', 25 * 1024 * 1024)
            self.scaling_tensor_reducer = _ScalingTensorReducer(scaling, self.process_group, cap)
            model_state.use_fp8_ddp = True
        self._anchor = torch.nn.Parameter(torch.empty(0, device=self.device if hasattr(self, 'device') else None))

    def forward(self, *inputs, **kwargs):
        if self.scaling_tensor_reducer is not None and torch.is_grad_enabled():
            self.scaling_tensor_reducer.sync = bool(getattr(self, 'require_backward_grad_sync', True))
            tensors = [(i, t) for i, t in enumerate(inputs) if torch.is_tensor(t)]
            anchor = self._anchor
            outs = _DDPSink.apply(self.scaling_tensor_reducer, anchor, anchor, *[t for _, t in tensors])
            inputs = list(inputs)
            for (i, _), o in zip(tensors, outs[1:]):
                inputs[i] = o
            inputs = tuple(inputs)
        return super().forward(*inputs, **kwargs)


def install():
    """Make ``torch.nn.parallel.DistributedDataParallel`` resolve to the FP8-aware class (as the reference does on import)."""
    torch.nn.parallel.DistributedDataParallel = FP8DistributedDataParallel


install()
