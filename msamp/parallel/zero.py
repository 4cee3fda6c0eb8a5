"""Sharded data parallelism for FP8 models (ZeRO stages 1/2 semantics, plus a replicated stage 0).

Ownership follows the reference's FP8 ZeRO optimizer (msamp/deepspeed/runtime/zero/fp8_stage_1_and_2.py:77-110):
whole tensors are assigned greedily to the least-loaded rank; the owner keeps the scaled-fp16 master
weight and the low-bit Adam moments; every rank keeps the e4m3 weights (flat buffer) and produces e4m3
weight gradients (flat buffer).  What differs is how data moves:

* both flat buffers live in symmetric memory, so one fused kernel per step replaces the per-parameter
  amax all-reduce (X12) and per-parameter ``ncclReduce`` (X13): each owner pulls its tensors from all
  peers over NVLink, dequantises with each peer's own scale, averages in fp32 and rounds once;
* after the partitioned LBAdam step one fused kernel casts each master to e4m3 and stores it straight
  into every peer's weight buffer with its ``scale_inv`` (replaces X14 + X15).

On backends without CUDA (gloo tests) the same algorithm runs with emulated collectives.
"""
import ctypes

import torch
import torch.distributed as dist

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingMeta, ScalingTensor
from msamp.common.utils.dist import DistUtil
from msamp.nn import ScalingParameter, model_state

E4M3 = Dtypes.kfloat8_e4m3


def partition_tensors(sizes, world):
    """Greedy whole-tensor partition: each tensor (in order) goes to the currently least-loaded rank.

    Returns ``owners`` (list of rank per tensor). Ties go to the lowest rank, so every process computes
    the same answer without communicating.
    """
    load = [0] * world
    owners = []
    for n in sizes:
        r = min(range(world), key=lambda k: (load[k], k))
        owners.append(r)
        load[r] += n
    return owners


def _pad16(n):
    return (n + 15) // 16 * 16


class ZeroShardedOptimizer:
    """Wraps an LB optimizer: reduce gradients to their owners, update the owned shard, publish the new weights.

    Args:
        model: model converted by ``msamp.initialize`` / ``LinearReplacer`` (FP8Linear weights are ScalingParameters).
        optimizer: the LBAdam/LBAdamW/DSAdam built for it.
        stage: 0 = replicated states (FP8 all-reduce), 1 or 2 = sharded master weights and moments.
        group: data-parallel process group.
        fuse_adam: stages 1 / 2: fold the FP8 gradient reduce-scatter into the first pass of the Adam kernel.
        overlap_comm: reduce the FP8 gradients bucket by bucket on a side stream while backward is still running (the
            reference reduces from backward hooks as well, msamp/deepspeed/runtime/zero/fp8_stage_1_and_2.py:378-443).
            The caller says which backward pass is the last of an optimizer step with ``reduce_in_backward(True)``.
        bucket_bytes: FP8 gradient bytes per bucket of the overlapped reduction.
    """
    def __init__(self, model, optimizer, stage=2, group=None, wait_seconds=5.0, model_parallel_group=None, fuse_adam=True,
                 overlap_comm=False, bucket_bytes=256 << 20):
        self.model, self.optimizer, self.stage, self.group = model, optimizer, stage, group
        self.world = DistUtil.get_world_size(group)
        self.rank = DistUtil.get_rank(group)
        self.wait_seconds = wait_seconds
        self.model_parallel_group = model_parallel_group    # gradient-norm clipping sums over it as well
        params = [p for p in model.parameters() if isinstance(p, ScalingParameter)]
        self.fp8_params = params
        # Expert (MoE) parameters carry ``allreduce = False`` (DeepSpeed's marker): every data-parallel rank holds different
        # experts, so they are neither reduced over the data-parallel group nor sharded; their gradient norm is summed
        # over the group like that of any parameter held by one rank only (reference: fp8/fused_optimizer.py:375-397).
        self.local_params = [p for p in model.parameters() if not isinstance(p, ScalingParameter) and getattr(p, 'allreduce', True) is False]
        if any(getattr(p, 'allreduce', True) is False for p in params):
            raise NotImplementedError('FP8 expert weights (ScalingParameter with allreduce=False) are not supported by the sharded optimizer')
        local_ids = {id(p) for p in self.local_params}
        self.hp_params = [p for p in model.parameters() if not isinstance(p, ScalingParameter) and id(p) not in local_ids]
        sizes = [p.numel() for p in params]
        self.owners = partition_tensors(sizes, self.world)
        offs = [0]
        for n in sizes:
            offs.append(offs[-1] + _pad16(n))
        self.offsets = offs
        self.n = len(params)
        self.device = params[0].device if params else torch.device('cpu')
        self.native = self.device.type == 'cuda' and self.world > 1
        self.sharded = stage >= 1    # with one rank this is plain FP8 weights + fp16 masters (the O3 layout)
        self._build_buffers()
        if self.sharded:
            self._shard_states()
        self._build_hp_buffers()
        # Stages 1 / 2 on the native path: the FP8 gradient reduce-scatter runs inside stage 1 of the fused Adam kernel
        # (each owner pulls its tensors' bytes from all ranks while it streams its own parameters and moments).
        self.fuse_adam = bool(fuse_adam) and self.native and self.sharded and hasattr(optimizer, '_reduce_in_step') \
            and getattr(optimizer, 'tensor_scale', False)
        if self.fuse_adam:
            self._fused_grads = {}
            for i, m in self.masters.items():
                p = self.fp8_params[i]
                # the reduced gradient's scale_inv lands in meta row 2 (row 0 is this rank's own contribution, which the
                # peers are still reading)
                meta = ScalingMeta(E4M3, scale=torch.ones((), device=self.device), scale_inv=self.g_meta_t[2, i:i + 1].view(()),
                                   amax=self.g_meta_t[1, i:i + 1], window_size=1)
                self._fused_grads[i] = ScalingTensor(p._grad_out, meta)
            self._reduce_desc = dict(index={id(m): i for i, m in self.masters.items()}, data_table=self.g_buf.table,
                                     meta_table=self.g_meta.table, world=self.world, rank=self.rank, n_tensors=self.n)

        self.overlap_comm = bool(overlap_comm) and self.native
        self._overlap_armed = False
        if self.overlap_comm:
            self._setup_overlap(bucket_bytes)

    # ------------------------------------------------------------------ overlapped reduction
    def _setup_overlap(self, bucket_bytes):
        """Buckets of FP8 parameters in the order their gradients appear (last layer first), the per-bucket work lists of
        the fused reduce kernel, and a hook on every parameter that launches a bucket once all of its gradients exist."""
        self.comm_stream = torch.cuda.Stream(device=self.device)
        chunk = 16384
        self.buckets = []    # dict(tensors=[i...], work_t, n_work, commit_t, n_commit)
        cur, size = [], 0
        for i in reversed(range(self.n)):
            cur.append(i)
            size += self.fp8_params[i].numel()
            if size >= bucket_bytes:
                self.buckets.append(cur)
                cur, size = [], 0
        if cur:
            self.buckets.append(cur)
        self.bucket_of = {}
        built = []
        for b, tensors in enumerate(self.buckets):
            work = []
            for i in tensors:
                self.bucket_of[i] = b
                if self.sharded and self.owners[i] != self.rank:
                    continue
                if not self.sharded and (i % self.world) != self.rank:
                    continue    # all-reduce flavour: the tensors of a bucket are dealt to the ranks in turn
                nb = _pad16(self.fp8_params[i].numel())
                work += [(i, c) for c in range((nb + chunk - 1) // chunk)]
            commit = [i for i in tensors if (not self.sharded) or self.owners[i] == self.rank]
            built.append(dict(
                tensors=tensors, n_work=len(work), n_commit=len(commit),
                work_t=torch.tensor(work if work else [(0, 0)], dtype=torch.int32, device=self.device).reshape(-1),
                commit_t=torch.tensor(commit if commit else [0], dtype=torch.int32, device=self.device)))
        self.buckets = built
        self._pending = [set() for _ in self.buckets]
        self._launched = [False] * len(self.buckets)
        for i, p in enumerate(self.fp8_params):
            p.register_backward_post_hook(self._make_overlap_hook(i))

    def _make_overlap_hook(self, i):
        def hook(*args, **kwargs):
            if not self._overlap_armed:
                return
            b = self.bucket_of[i]
            self._pending[b].discard(i)
            if not self._pending[b] and not self._launched[b]:
                self._launch_bucket(b)
        return hook

    def reduce_in_backward(self, enabled=True):
        """Arm (or disarm) the overlapped reduction for the next backward pass: call with True right before the last
        backward of an optimizer step (gradient accumulation: earlier micro-batches must not be reduced)."""
        if not self.overlap_comm:
            return
        self._overlap_armed = bool(enabled)
        if enabled:
            self._pending = [set(b['tensors']) for b in self.buckets]
            self._launched = [False] * len(self.buckets)

    def _launch_bucket(self, b):
        from msamp.ops import native
        bucket = self.buckets[b]
        self._launched[b] = True
        self.comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.comm_stream):
            epoch = self.flags.next_epoch()
            # 64 CTAs: the kernel shares the GPU with the GEMMs of the remaining backward pass
            native.check(
                native.lib().msamp_symm_grad_reduce(
                    self.g_buf.table, self.g_meta.table, self.flags.table, native.ptr(self.offsets_t), native.ptr(bucket['work_t']),
                    bucket['n_work'], self.n, self.rank, self.world, ctypes.c_uint(epoch), 0 if self.sharded else 1,
                    ctypes.c_double(self.wait_seconds), 64, native.stream()
                ), 'symm_grad_reduce(bucket)'
            )
            native.check(
                native.lib().msamp_symm_commit_meta(native.ptr(self.g_meta_t), self.n, native.ptr(bucket['commit_t']), bucket['n_commit'],
                                                    native.stream()), 'symm_commit_meta'
            )

    def _finish_overlapped(self):
        """Launch what backward did not (parameters without a gradient keep their bucket open) and join the side stream.
        Returns True if the FP8 gradients were reduced this way."""
        if not (self.overlap_comm and self._overlap_armed):
            return False
        for b in range(len(self.buckets)):
            if not self._launched[b]:
                self._launch_bucket(b)
        torch.cuda.current_stream().wait_stream(self.comm_stream)
        self._overlap_armed = False
        return True

    # ------------------------------------------------------------------ set-up
    def _alloc(self, nbytes):
        if self.native:
            from msamp.parallel.symm import SymmetricBuffer
            return SymmetricBuffer(max(nbytes, 16), self.group)
        return None

    def _build_buffers(self):
        total = self.offsets[-1]
        n = self.n
        if self.native:
            from msamp.parallel.symm import FlagPad
            self.g_buf = self._alloc(total)
            self.g_meta = self._alloc(3 * n * 4)
            self.flags = FlagPad(self.group)
            g_flat = self.g_buf.view(torch.uint8)
            g_meta = self.g_meta.view(torch.float32).view(3, n)
        else:
            g_flat = torch.zeros(max(total, 1), dtype=torch.uint8, device=self.device)
            g_meta = torch.zeros(3, max(n, 1), dtype=torch.float32, device=self.device)
        g_meta[0].fill_(1.0)
        self.g_flat, self.g_meta_t = g_flat, g_meta
        # gradient metas: re-home scale_inv / amax of every layer's 'wgrad' meta into the meta rows
        self.meta_index = []
        for i, p in enumerate(self.fp8_params):
            meta = p._scaling_metas['wgrad']
            if meta.window_size != 1:
                raise RuntimeError('sharded FP8 gradients need a wgrad window of 1')
            was_locked, meta.locked = meta.locked, False
            si, am = g_meta[0, i:i + 1].view(()), g_meta[1, i:i + 1]
            si.copy_(meta.scale_inv)
            am.copy_(meta.amax)
            meta.scale_inv, meta.amax = si, am
            meta.locked = was_locked
            p._grad_out = g_flat[self.offsets[i]:self.offsets[i] + p.numel()].view(p.shape)
        # the metas no longer alias model_state's flat wgrad buffers; tell model_state so its aliasing check passes
        flat = model_state.flattened_scaling_metas
        if flat is not None and 'wgrad' in flat:
            flat['wgrad'] = dict(flat['wgrad'], scales_inv=g_meta[0], amaxs=g_meta[1].view(-1, 1), _external=True)
        # every offset a kernel will add to a (peer) base pointer, checked against the buffer it indexes: the kernels read
        # 16-byte vectors up to the padded end of a tensor and three fp32 meta rows of n entries
        for i, p in enumerate(self.fp8_params):
            lo, hi = self.offsets[i], self.offsets[i] + _pad16(p.numel())
            if lo % 16 or hi > g_flat.numel() or (i + 1 < len(self.offsets) and hi > self.offsets[i + 1]):
                raise RuntimeError(f'gradient buffer layout: tensor {i} covers [{lo}, {hi}) of {g_flat.numel()} bytes')
        if g_meta.numel() < 3 * max(n, 1):
            raise RuntimeError('gradient meta rows are too short')
        work = []
        chunk = 16384
        for i, p in enumerate(self.fp8_params):
            if self.owners[i] == self.rank:
                nb = _pad16(p.numel())
                work += [(i, c) for c in range((nb + chunk - 1) // chunk)]
        self.n_work = len(work)
        self.work_t = torch.tensor(work if work else [(0, 0)], dtype=torch.int32, device=self.device).reshape(-1)
        self.offsets_t = torch.tensor(self.offsets, dtype=torch.int64, device=self.device)
        self.owned = [i for i in range(n) if self.owners[i] == self.rank]
        self.owned_t = torch.tensor(self.owned if self.owned else [0], dtype=torch.int32, device=self.device)
        self.all_t = torch.arange(max(n, 1), dtype=torch.int32, device=self.device)

    def _shard_states(self):
        """FP8 weights in a flat (symmetric) buffer on every rank; scaled-fp16 masters and moments only on the owner."""
        total, n = self.offsets[-1], self.n
        if self.native:
            self.w_buf = self._alloc(total)
            self.w_meta = self._alloc(3 * n * 4)
            w_flat = self.w_buf.view(torch.uint8)
            w_meta = self.w_meta.view(torch.float32).view(3, n)
        else:
            w_flat = torch.zeros(max(total, 1), dtype=torch.uint8, device=self.device)
            w_meta = torch.zeros(3, max(n, 1), dtype=torch.float32, device=self.device)
        self.w_flat, self.w_meta_t = w_flat, w_meta
        # masters of the owned tensors share one padded fp16 buffer so that 16-element vector reads never leave it
        owned_total = sum(_pad16(self.fp8_params[i].numel()) for i in self.owned)
        self.master_flat = torch.zeros(max(owned_total, 1), dtype=torch.float16, device=self.device)
        self.masters = {}
        replace = {}
        moff = 0
        for i, p in enumerate(self.fp8_params):
            n_el = p.numel()
            if self.owners[i] == self.rank:
                src = p if p.qtype == Dtypes.kfloat16 else p.cast(Dtypes.kfloat16)
                mval = self.master_flat[moff:moff + n_el].view(p.shape)
                mval.copy_(src.value)
                mmeta = ScalingMeta(Dtypes.kfloat16, window_size=1, device=self.device)
                mmeta.copy_(src.meta)
                master = ScalingParameter(ScalingTensor(mval, mmeta), requires_grad=True)
                self.masters[i] = master
                replace[id(p)] = master
                moff += _pad16(n_el)
            else:
                replace[id(p)] = None
            # the model-side weight becomes e4m3 in the flat buffer, its scale_inv/amax in the meta rows
            q = p if p.qtype == E4M3 else p.cast(E4M3)
            view = w_flat[self.offsets[i]:self.offsets[i] + n_el].view(p.shape)
            view.copy_(q.value)
            si, am = w_meta[0, i:i + 1].view(()), w_meta[1, i:i + 1]
            si.copy_(q.meta.scale_inv)
            am.copy_(q.meta.amax)
            new_meta = ScalingMeta(E4M3, scale=torch.reciprocal(si), scale_inv=si, amax=am, window_size=1)
            p.value = view
            p.meta = new_meta
            p._fp8_cache = None
        # rebind the optimizer's groups: owned FP8 params -> masters, others dropped
        for group in self.optimizer.param_groups:
            new = []
            for p in group['params']:
                if id(p) in replace:
                    if replace[id(p)] is not None:
                        new.append(replace[id(p)])
                else:
                    new.append(p)
            group['params'] = new
        self.optimizer.state.clear()
        if self.native:
            ptrs = [0] * n
            sinvs = [0] * n
            amaxs = [0] * n
            for i, m in self.masters.items():
                ptrs[i], sinvs[i], amaxs[i] = m.value.data_ptr(), m.meta.scale_inv.data_ptr(), m.meta.amax.data_ptr()
            self.master_ptrs = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
            self.master_sinvs = torch.tensor(sinvs, dtype=torch.int64, device=self.device)
            self.master_amaxs = torch.tensor(amaxs, dtype=torch.int64, device=self.device)

    # ------------------------------------------------------------------ step
    def _reduce_fp8_grads(self):
        broadcast = 0 if self.sharded else 1
        if self.native:
            from msamp.ops import native
            epoch = self.flags.next_epoch()
            native.check(
                native.lib().msamp_symm_grad_reduce(
                    self.g_buf.table, self.g_meta.table, self.flags.table, native.ptr(self.offsets_t), native.ptr(self.work_t), self.n_work,
                    self.n, self.rank, self.world, ctypes.c_uint(epoch), broadcast, ctypes.c_double(self.wait_seconds), 0, native.stream()
                ), 'symm_grad_reduce'
            )
            which = self.all_t if broadcast else self.owned_t
            count = self.n if broadcast else len(self.owned)
            native.check(
                native.lib().msamp_symm_commit_meta(native.ptr(self.g_meta_t), self.n, native.ptr(which), count, native.stream()),
                'symm_commit_meta'
            )
            return
        if self.world == 1:
            return
        self._emulated_reduce(broadcast)

    def _emulated_reduce(self, broadcast):
        """Same arithmetic as the fused kernel, with gloo/NCCL collectives: gather bytes + metas, average in fp32, round once."""
        from msamp.ops import cast as _k
        from msamp.common.dtype import Floating
        flats = [torch.empty_like(self.g_flat) for _ in range(self.world)]
        metas = [torch.empty_like(self.g_meta_t) for _ in range(self.world)]
        dist.all_gather(flats, self.g_flat, group=self.group)
        dist.all_gather(metas, self.g_meta_t.contiguous(), group=self.group)
        for i, p in enumerate(self.fp8_params):
            if not broadcast and self.owners[i] != self.rank:
                continue
            lo, hi = self.offsets[i], self.offsets[i] + p.numel()
            acc = torch.zeros(p.numel(), dtype=torch.float32, device=self.device)
            amax = torch.zeros((), device=self.device)
            for r in range(self.world):
                acc += flats[r][lo:hi].view(torch.float8_e4m3fn).float() * (metas[r][0, i] / self.world)
                amax = torch.maximum(amax, torch.nan_to_num(metas[r][1, i], nan=float('inf')))
            scale = _k.compute_scale(amax, torch.ones((), device=self.device), Floating.qfp_max[E4M3])
            self.g_flat[lo:hi] = _k._emulate_to_fp8(acc, scale, E4M3)
            self.g_meta_t[0, i] = 1.0 / scale

    # ------------------------------------------------------------------ high-precision parameters
    def _build_hp_buffers(self):
        """Everything that is not an FP8 weight goes through ``HighPrecisionShards``: replicated with one flat gradient
        all-reduce per dtype at stage 0, sharded like stock ZeRO (owner per tensor, reduce-scatter, all-gather) at stages 1 / 2."""
        from msamp.parallel.hp_shard import HighPrecisionShards
        self.hp = HighPrecisionShards(self.hp_params, self.group, shard=self.sharded, device=self.device)
        self.hp.bind_optimizer(self.optimizer)
        self.hp_owner, self.hp_layout = self.hp.owner, self.hp.layout

    def _owned_hp(self):
        return self.hp.owned()

    def _reduce_hp_grads(self):
        self.hp.reduce_grads()

    def _gather_hp_params(self):
        """Publish the owners' updated high-precision parameters to every rank (stages 1 / 2)."""
        self.hp.gather_params()

    def _clear_hp_grads(self):
        self.hp.clear_grads()

    def _publish_weights(self):
        if self.native:
            from msamp.ops import native
            epoch = self.flags.next_epoch()
            native.check(
                native.lib().msamp_symm_cast_bcast(
                    self.w_buf.table, self.w_meta.table, self.flags.table, native.ptr(self.offsets_t), native.ptr(self.work_t), self.n_work,
                    self.n, native.ptr(self.master_ptrs), native.ptr(self.master_sinvs), native.ptr(self.master_amaxs), self.rank, self.world,
                    ctypes.c_uint(epoch), ctypes.c_double(self.wait_seconds), native.stream()
                ), 'symm_cast_bcast'
            )
        else:
            from msamp.ops import cast as _k
            for i, m in self.masters.items():
                p = self.fp8_params[i]
                # master value is w * s_m: one pass rescales by rule(amax) / s_m, rounds to e4m3 and stores 1 / rule(amax)
                new_scale = _k.compute_scale(m.meta.amax[0], torch.ones((), device=self.device), 448.0)
                factor = new_scale * m.meta.scale_inv
                _k.cast_to_fp8(m.value, E4M3, factor, out=p.value.view(-1))
                self.w_meta_t[0, i] = torch.reciprocal(new_scale)
                self.w_meta_t[1, i] = m.meta.amax[0]
            if self.world > 1:
                flats = [torch.empty_like(self.w_flat) for _ in range(self.world)]
                metas = [torch.empty_like(self.w_meta_t) for _ in range(self.world)]
                dist.all_gather(flats, self.w_flat, group=self.group)
                dist.all_gather(metas, self.w_meta_t.contiguous(), group=self.group)
                for i, p in enumerate(self.fp8_params):
                    r = self.owners[i]
                    if r != self.rank:
                        lo, hi = self.offsets[i], self.offsets[i] + p.numel()
                        self.w_flat[lo:hi] = flats[r][lo:hi]
                        self.w_meta_t[:2, i] = metas[r][:2, i]
        for p in self.fp8_params:
            torch.autograd.graph.increment_version(p.value)

    def reduce_and_step(self, clip_grad=0.0):
        """Call after backward: exchange gradients, update the owned shard, publish weights, clear gradients."""
        overlapped = self._finish_overlapped()    # gradients already reduced bucket by bucket during backward
        fused = self.fuse_adam and clip_grad <= 0 and not overlapped    # clipping needs the reduced gradients' norm before the update
        if fused:
            # one cross-rank barrier (all gradients and metas are written), then reduce-scatter + Adam in one kernel
            self.flags.barrier(slot=3, limit_seconds=self.wait_seconds)
            self._reduce_hp_grads()
            for i, m in self.masters.items():
                m.grad = self._fused_grads[i] if self.fp8_params[i].grad is not None else None
            self.optimizer._reduce_in_step = self._reduce_desc
            try:
                self.optimizer.step()
            finally:
                self.optimizer._reduce_in_step = None
        else:
            if not overlapped:
                self._reduce_fp8_grads()
            self._reduce_hp_grads()
            if self.sharded:
                for i, m in self.masters.items():
                    p = self.fp8_params[i]
                    m.grad = p.grad
            if clip_grad > 0:
                self._clip(clip_grad)
            self.optimizer.step()
        if self.sharded:
            self._publish_weights()
            self._gather_hp_params()
            for m in self.masters.values():
                m.grad = None
        for p in self.fp8_params:
            p.grad = None
        if self.hp_layout:
            self._clear_hp_grads()

    def _clip(self, max_norm):
        """Global-norm clipping: one multi-tensor launch for this rank's share of the squared norm, the cross-rank sums,
        one launch that scales (FP8 gradients through their ``scale_inv``)."""
        from msamp.ops import multi_tensor as _mt
        owned = list(self.masters.values()) if self.sharded else self.fp8_params
        mp_group = getattr(self, 'model_parallel_group', None)
        mp_rank = dist.get_rank(mp_group) if mp_group is not None else 0
        hp = self._owned_hp() if (self.sharded and self.world > 1) else self.hp_params
        counted = [p.grad for p in owned if p.grad is not None]
        clipped = list(counted)
        for p in hp:
            if p.grad is None:
                continue
            clipped.append(p.grad)
            if mp_group is not None and mp_rank != 0 and not getattr(p, 'tensor_model_parallel', False):
                continue    # replicated over the model-parallel group: counted on its first rank only
            counted.append(p.grad)
        local = [p.grad for p in self.local_params if p.grad is not None]
        clipped += local
        if not self.sharded and self.world > 1:
            # replicated states: every rank holds every gradient, so the local sum already is the data-parallel total;
            # only the expert parameters (different on every rank) have to be summed over the group
            stats = _mt.grad_sumsq(counted, tag='zero_norm')
            if self.local_params:
                extra = _mt.grad_sumsq(local, out=torch.zeros_like(stats), tag='zero_norm_local')
                dist.all_reduce(extra, group=self.group)
                stats = stats + extra
        else:
            stats = _mt.grad_sumsq(counted + local, tag='zero_norm')
            if self.world > 1:
                dist.all_reduce(stats, group=self.group)
        if stats.device != self.device:
            stats = stats.to(self.device)
        if mp_group is not None and dist.get_world_size(mp_group) > 1:
            # the model-parallel ranks hold different shards of the model: one norm, one clip coefficient for all
            dist.all_reduce(stats, group=mp_group)
        _mt.clip_by_sumsq(clipped, stats[0:1], max_norm, tag='zero_clip')
        return stats[0].sqrt()

    # ------------------------------------------------------------------ checkpoint
    def _master_groups(self):
        """This rank's master weights as ``[[masters of param group 0], [masters of param group 1], ...]`` in the order of
        ``optimizer.param_groups`` - the nesting of ``single_partition_of_fp8_groups`` in the reference's checkpoint
        (msamp/deepspeed/runtime/zero/fp8_stage_1_and_2.py:937-960)."""
        mine = {id(m) for m in getattr(self, 'masters', {}).values()}
        return [[p for p in g['params'] if id(p) in mine] for g in self.optimizer.param_groups]

    def state_dict(self):
        """Inner optimizer state plus this rank's master weights, under the reference's key name and nesting."""
        return {
            'optimizer_state_dict': self.optimizer.state_dict(),
            'single_partition_of_fp8_groups': [[m.detach() for m in group] for group in self._master_groups()],
            'partition_count': self.world,
            'zero_stage': self.stage,
        }

    def load_state_dict(self, sd):
        if sd.get('partition_count', self.world) != self.world:
            raise ValueError('loading a sharded optimizer state needs the same data-parallel size')
        self.optimizer.load_state_dict(sd['optimizer_state_dict'])
        saved = sd['single_partition_of_fp8_groups']
        groups = self._master_groups()
        if saved and not isinstance(saved[0], (list, tuple)):
            # legacy layout of this library: one flat list in ascending tensor index
            flat_masters = [self.masters[i] for i in sorted(getattr(self, 'masters', {}))]
            if len(saved) != len(flat_masters):
                raise ValueError(f'checkpoint holds {len(saved)} FP8 master weights, this rank owns {len(flat_masters)}')
            pairs = list(zip(flat_masters, saved))
        else:
            if len(saved) != len(groups) or any(len(a) != len(b) for a, b in zip(saved, groups)):
                raise ValueError('single_partition_of_fp8_groups does not match the optimizer\'s parameter groups: '
                                 f'{[len(g) for g in saved]} vs {[len(g) for g in groups]}')
            pairs = [(m, t) for g_m, g_t in zip(groups, saved) for m, t in zip(g_m, g_t)]
        for master, tensor in pairs:
            master.copy_(tensor.to(device=self.device))
        if self.sharded:
            self._publish_weights()

    def _rehome(self):
        """Move everything that aliases the symmetric buffers (the FP8 weights and their scale_inv / amax, the wgrad metas'
        scale_inv / amax, the gradient views, model_state's flat wgrad tables) into ordinary device memory, values kept.
        Without this the model, and the process-wide meta registry that is re-flattened whenever another model registers,
        would keep reading memory that ``close()`` is about to free."""
        for p in self.fp8_params:
            metas = getattr(p, '_scaling_metas', None) or {}
            meta = metas.get('wgrad')
            if meta is not None:
                was_locked, meta.locked = meta.locked, False
                meta.scale_inv, meta.amax = meta.scale_inv.clone(), meta.amax.clone()
                meta.locked = was_locked
            p._grad_out = None
            if p.grad is not None:
                p.grad = None
            if self.sharded and getattr(self, 'w_buf', None) is not None:
                p.value = p.value.clone()
                p.meta.scale_inv, p.meta.amax = p.meta.scale_inv.clone(), p.meta.amax.clone()
                p._fp8_cache = None
        self._fused_grads = {}
        flat = model_state.flattened_scaling_metas
        if flat is not None and flat.get('wgrad', {}).get('_external'):
            model_state.reflatten()
        self.g_flat = self.g_meta_t = self.w_flat = self.w_meta_t = None

    def close(self):
        """Release the symmetric (IPC-shared) buffers.  Collective: every rank of the group calls it, after its last step.
        The model keeps its FP8 weights (copied to ordinary memory); the optimizer can no longer step."""
        if self.native and getattr(self, 'g_buf', None) is not None:
            torch.cuda.synchronize(self.device)
            self._rehome()
            torch.cuda.synchronize(self.device)
        for name in ('g_buf', 'g_meta', 'w_buf', 'w_meta', 'flags'):
            buf = getattr(self, name, None)
            if buf is not None and hasattr(buf, 'close'):
                if self.world > 1:
                    dist.barrier(group=self.group)    # nobody may still be reading this rank's memory
                buf.close()
                setattr(self, name, None)

    # ------------------------------------------------------------------ elastic checkpoint (any data-parallel degree)
    def elastic_state_dict(self):
        """State of this rank keyed by *global* tensor index, for resuming at another data-parallel degree.

        ``{'fp8': {i: {'master', 'state'}}, 'hp': {k: state}, 'param_groups': [...]}``: ``i`` indexes the model's FP8
        parameters in ``model.parameters()`` order, ``k`` the remaining parameters (their states are replicated, so
        any one rank's copy serves).  ``consolidate_elastic_state`` merges the dictionaries of all ranks.
        The reference cannot change the degree on resume (msamp/deepspeed/runtime/zero/fp8_stage_1_and_2.py:1007-1017).
        """
        fp8 = {}
        for i, master in getattr(self, 'masters', {}).items():
            fp8[i] = {'master': master.detach(), 'state': dict(self.optimizer.state.get(master, {}))}
        hp = {k: dict(self.optimizer.state.get(p, {})) for k, p in enumerate(self.hp_params) if p in self.optimizer.state}    # owned ones only when sharded
        groups = [{k: v for k, v in g.items() if k != 'params'} for g in self.optimizer.param_groups]
        return {'fp8': fp8, 'hp': hp, 'param_groups': groups, 'num_fp8': self.n, 'partition_count': self.world}

    @staticmethod
    def consolidate_elastic_state(states):
        """Merge the ``elastic_state_dict`` of every rank of the saving job into one dictionary."""
        out = {'fp8': {}, 'hp': {}, 'param_groups': states[0]['param_groups'], 'num_fp8': states[0]['num_fp8'], 'partition_count': 0}
        for sd in states:
            out['fp8'].update(sd['fp8'])
            for k, st in sd['hp'].items():
                out['hp'].setdefault(k, st)
        missing = [i for i in range(out['num_fp8']) if i not in out['fp8']]
        if missing:
            raise ValueError(f'elastic state is incomplete: no owner state for FP8 tensors {missing}')
        return out

    def load_elastic_state_dict(self, full):
        """Take from a consolidated elastic state what this rank owns under the *current* partition."""
        if not self.sharded:
            raise RuntimeError('elastic states belong to sharded optimizers (stage >= 1)')
        if full['num_fp8'] != self.n:
            raise ValueError(f"the state holds {full['num_fp8']} FP8 tensors, the model has {self.n}")

        def to_dev(v):
            return v.to(self.device) if hasattr(v, 'to') else v

        for i, master in self.masters.items():
            entry = full['fp8'][i]
            master.copy_(to_dev(entry['master']))
            if entry['state']:
                self.optimizer.state[master] = {k: to_dev(v) for k, v in entry['state'].items()}
        for k, p in enumerate(self.hp_params):
            if k in full['hp'] and full['hp'][k] and self.hp_owner[k] == self.rank:
                self.optimizer.state[p] = {key: to_dev(v) for key, v in full['hp'][k].items()}
        for g, saved in zip(self.optimizer.param_groups, full['param_groups']):
            g.update(saved)
        self._publish_weights()

