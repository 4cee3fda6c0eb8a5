"""FP8 DistributedDataParallel.

A drop-in subclass of torch's DDP.  High-precision parameters go through torch's own reducer;
FP8Linear weights (DDP-ignored ScalingParameters) are handled by ``_ScalingTensorReducer``: they are
packed in reverse registration order into byte-capped buckets, and when the last gradient of a bucket
arrives the bucket's amax values are MAX-reduced, a common scale is derived (pre-scaled by 1/sqrt(W)
against overflow of the sum), the gradients are quantised to e4m3 into one flat buffer, and the buffer
is SUM-reduced as FP8 numbers asynchronously; ``scale_inv`` is divided by W so the result is the mean.
``_DDPSink`` resets the bucket bookkeeping in forward and waits for the collectives at the end of backward.
(reference: msamp/nn/distributed.py:18-264)

On CUDA with NCCL (up to 8 ranks on one NVLink domain) a bucket takes the fused path instead: ONE multi-tensor launch
quantises the bucket's gradients into a flat buffer in symmetric memory, each rank with its own in-time scale (the amax
comes from the wgrad GEMM epilogue, so there is no amax collective), and ONE launch of the fused all-reduce kernel
(``msamp_symm_grad_reduce``, broadcast flavour) pulls every peer's bytes over NVLink, dequantises each with that peer's
scale, averages in fp32, rounds once and writes the result to every rank - on the side stream, overlapped with the rest
of backward.  The NCCL path remains for gloo / CPU and as the oracle of the tests.
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
        self.fused = False
        self._setup_fused()
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

    def _setup_fused(self):
        """Symmetric buffers, per-bucket work lists and re-homed gradient metas for the fused all-reduce kernel."""
        import os
        world = dist.get_world_size(self.process_group) if dist.is_initialized() else 1
        if (self.device.type != 'cuda' or world < 2 or not self.parameters or dist.get_backend(self.process_group) != 'nccl'
                or os.environ.get('MSAMP_DDP_FUSED', '1') == '0'):
            return
        from msamp.ops import native
        from msamp.parallel.symm import FlagPad, SymmetricBuffer
        if world > native.lib().msamp_symm_max_ranks():
            return
        self.rank, self.world = dist.get_rank(self.process_group), world
        n = len(self.parameters)
        # flat layout: buckets in order, tensors of a bucket in bucket order, every tensor padded to 16 bytes
        self.tensor_offset = [0] * (n + 1)    # indexed by position in the flat order
        self.flat_index = {}                  # parameter id -> position in the flat order
        off = 0
        order = [pid for b in sorted(self.bucket_to_param_ids) for pid in self.bucket_to_param_ids[b]]
        for k, pid in enumerate(order):
            self.flat_index[pid] = k
            self.tensor_offset[k] = off
            off += (self.parameters[pid].numel() + 15) // 16 * 16
        self.tensor_offset[n] = off
        self.g_buf = SymmetricBuffer(max(off, 16), self.process_group)
        self.g_meta = SymmetricBuffer(3 * n * 4, self.process_group)
        self.flags = FlagPad(self.process_group)
        self.g_flat = self.g_buf.view(torch.uint8)
        self.g_meta_t = self.g_meta.view(torch.float32).view(3, n)
        self.g_meta_t[0].fill_(1.0)
        self.offsets_t = torch.tensor(self.tensor_offset, dtype=torch.int64, device=self.device)
        chunk = native.lib().msamp_symm_chunk_bytes()
        self.bucket_work, self.bucket_tensors = {}, {}
        turn = 0
        for b, pids in self.bucket_to_param_ids.items():
            work, tensors = [], []
            for pid in pids:
                k = self.flat_index[pid]
                tensors.append(k)
                nbytes = self.tensor_offset[k + 1] - self.tensor_offset[k]
                for c in range((nbytes + chunk - 1) // chunk):
                    if turn % world == self.rank:    # chunks are dealt to the ranks in turn; each reduces its share for everybody
                        work.append((k, c))
                    turn += 1
            self.bucket_work[b] = (torch.tensor(work if work else [(0, 0)], dtype=torch.int32, device=self.device).reshape(-1), len(work))
            self.bucket_tensors[b] = torch.tensor(tensors, dtype=torch.int32, device=self.device)
        # the gradient metas' scale_inv / amax move into the symmetric meta rows, where the peers can read them
        for pid, p in enumerate(self.parameters):
            meta = p._scaling_metas['wgrad'] if hasattr(p, '_scaling_metas') else None
            if meta is None or meta.window_size != 1:
                return    # not an FP8Linear weight: keep the NCCL path
        for pid, p in enumerate(self.parameters):
            k = self.flat_index[pid]
            meta = p._scaling_metas['wgrad']
            was_locked, meta.locked = meta.locked, False
            si, am = self.g_meta_t[0, k:k + 1].view(()), self.g_meta_t[1, k:k + 1]
            si.copy_(meta.scale_inv)
            am.copy_(meta.amax)
            meta.scale_inv, meta.amax = si, am
            meta.locked = was_locked
        flat = model_state.flattened_scaling_metas
        if flat is not None and 'wgrad' in flat:
            # the metas no longer alias model_state's flat wgrad buffers; point its aliasing check at their new home
            flat['wgrad'] = dict(flat['wgrad'], scales_inv=self.g_meta_t[0], amaxs=self.g_meta_t[1].view(-1, 1), _external=True)
        self.fused = True

    def _reduce_bucket_fused(self, bucket):
        import ctypes
        from msamp.ops import multi_tensor as _mt
        from msamp.ops import native
        pids = self.bucket_to_param_ids[bucket]
        params = [self.parameters[pid] for pid in pids]
        self.reduction_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.reduction_stream):
            srcs, dsts, scales, sinvs, amaxs, metas = [], [], [], [], [], []
            for pid, p in zip(pids, params):
                g = p.grad
                if isinstance(g, ScalingTensor):
                    raise RuntimeError('FP8 DDP expects high-precision gradients carrying a .meta (set model_state.use_fp8_ddp)')
                k = self.flat_index[pid]
                meta = p._scaling_metas['wgrad']
                if getattr(g, 'meta', None) is not meta:
                    _k.amax(g, out=meta.amax[0])    # a gradient that did not come from the wgrad GEMM epilogue
                g = g.contiguous()
                g.record_stream(self.reduction_stream)
                lo = self.tensor_offset[k]
                srcs.append(g)
                dsts.append(self.g_flat[lo:lo + g.numel()])
                scales.append(meta.scale)
                sinvs.append(meta.scale_inv)
                amaxs.append(meta.amax[0])
                metas.append(meta)
            _mt.cast_to_fp8_multi(srcs, dsts, E4M3, scales, sinvs, amax_ins=amaxs, tag=f'fp8_ddp_bucket{bucket}')
            work_t, n_work = self.bucket_work[bucket]
            n = len(self.parameters)
            native.check(
                native.lib().msamp_symm_grad_reduce(
                    self.g_buf.table, self.g_meta.table, self.flags.table, native.ptr(self.offsets_t), native.ptr(work_t), n_work, n,
                    self.rank, self.world, ctypes.c_uint(self.flags.next_epoch()), 1, ctypes.c_double(5.0), 64, native.stream()    # 64 CTAs: it overlaps backward
                ), 'symm_grad_reduce'
            )
            tensors = self.bucket_tensors[bucket]
            native.check(
                native.lib().msamp_symm_commit_meta(native.ptr(self.g_meta_t), n, native.ptr(tensors), tensors.numel(), native.stream()),
                'symm_commit_meta'
            )
            for p, dst, meta in zip(params, dsts, metas):
                p.grad = ScalingTensor(dst.view(p.shape), meta)

    def close(self):
        """Release the symmetric buffers of the fused path (collective over the group)."""
        if self.fused:
            torch.cuda.synchronize()
            # the wgrad metas' scale_inv / amax and model_state's flat wgrad tables alias the symmetric meta rows: move them
            # into ordinary memory first (values kept), or the next re-flattening of the registry would read freed memory
            for p in self.parameters:
                meta = p._scaling_metas['wgrad'] if hasattr(p, '_scaling_metas') else None
                if meta is not None:
                    was_locked, meta.locked = meta.locked, False
                    meta.scale_inv, meta.amax = meta.scale_inv.clone(), meta.amax.clone()
                    meta.locked = was_locked
                if isinstance(p.grad, ScalingTensor):
                    p.grad = None
            flat = model_state.flattened_scaling_metas
            if flat is not None and flat.get('wgrad', {}).get('_external'):
                model_state.reflatten()
            self.g_meta_t = None
            torch.cuda.synchronize()
            dist.barrier(group=self.process_group)
            for buf in (self.g_buf, self.g_meta, self.flags):
                buf.close()
            self.fused = False

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
        if self.fused:
            return self._reduce_bucket_fused(bucket)
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
