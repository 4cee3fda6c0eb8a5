"""A small training-step driver used by the benchmark, the examples and the tests.

One call of ``step(tokens, labels)`` runs forward, backward, the gradient exchange of the chosen
data-parallel flavour and the optimizer update, and returns the (device-resident) loss.
"""
import torch
import torch.distributed as dist

from msamp.common.tensor import ScalingTensor, TensorDist
from msamp.common.utils.dist import DistUtil


class DataParallelTrainer:
    """Replicated data parallelism (``zero_stage=0``) or sharded optimizer states (``zero_stage=1/2``).

    FP8 weight gradients already share one scale across ranks (their amax is MAX-reduced when they
    are quantised), so they are summed as FP8 numbers and averaged by dividing ``scale_inv``;
    high-precision gradients are averaged in flat buckets.
    """
    def __init__(self, model, optimizer, zero_stage=0, group=None, clip_grad=0.0, bucket_elems=64 * 1024 * 1024, after_backward=None,
                 heartbeat=None, model_parallel_group=None, overlap_comm=False):
        self.model = model
        # msamp.utils.Heartbeat (optional): checked before every step, so a rank that went silent between steps raises
        # RankFailure on the others before they enter a collective or a fused kernel that would wait for it
        self.heartbeat = heartbeat
        # tensor / pipeline parallel ranks hold different shards: gradient clipping needs the norm over them too
        self.model_parallel_group = model_parallel_group
        # called after backward and before any gradient is reduced (e.g. ParallelGPT.allreduce_sequence_parallel_grads)
        self.after_backward = after_backward
        self.optimizer = optimizer
        self.group = group
        self.world = DistUtil.get_world_size(group)
        self.clip_grad = clip_grad
        self.bucket_elems = bucket_elems
        self.zero = None
        if zero_stage and self.world > 1:
            from msamp.parallel.zero import ZeroShardedOptimizer
            self.zero = ZeroShardedOptimizer(model, optimizer, stage=zero_stage, group=group, model_parallel_group=model_parallel_group,
                                             overlap_comm=overlap_comm)

    def _sync_grads(self):
        if self.world == 1:
            return
        fp8, hp = [], []
        for p in self.model.parameters():
            g = p.grad
            if g is None:
                continue
            (fp8 if isinstance(g, ScalingTensor) else hp).append(g)
        TensorDist.all_reduce_avg(fp8, bucket_size=self.bucket_elems, group=self.group)
        by_dtype = {}
        for g in hp:
            by_dtype.setdefault(g.dtype, []).append(g)
        for grads in by_dtype.values():
            flat = torch.cat([g.reshape(-1) for g in grads])
            dist.all_reduce(flat, group=self.group)
            flat.div_(self.world)
            off = 0
            for g in grads:
                n = g.numel()
                g.copy_(flat[off:off + n].view_as(g))
                off += n

    def step(self, *inputs):
        return self.step_micro_batches([inputs])

    def step_micro_batches(self, micro_batches):
        """One optimizer step over several micro-batches (gradient accumulation): every micro-batch runs forward and
        backward with its loss divided by their number, FP8 weight gradients accumulate in FP8 with a fresh scale per
        addition, and the gradient exchange happens once.  Returns the mean loss."""
        if self.heartbeat is not None:
            self.heartbeat.check()
        self.optimizer.zero_grad(set_to_none=True)
        k = len(micro_batches)
        total = None
        for n_mb, inputs in enumerate(micro_batches):
            if self.zero is not None and n_mb == k - 1:
                self.zero.reduce_in_backward(True)    # the last backward of the step may reduce gradients as they appear
            loss = self.model(*inputs)
            if k > 1:
                loss = loss / k
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        loss = total
        if self.after_backward is not None:
            self.after_backward()
        if self.zero is not None:
            self.zero.reduce_and_step(clip_grad=self.clip_grad)
        else:
            self._sync_grads()
            if self.clip_grad > 0 and self.model_parallel_group is not None:
                from msamp.megatron.optimizer.clip_grads import clip_grad_norm_fp32
                first = dist.get_rank(self.model_parallel_group) == 0
                params = [p for p in self.model.parameters() if p.grad is not None]
                counted = [p.grad for p in params if first or getattr(p, 'tensor_model_parallel', False)]
                clip_grad_norm_fp32(params, counted, self.clip_grad, 2, model_parallel_group=self.model_parallel_group)
            elif self.clip_grad > 0:
                from msamp.nn import clip_grad_norm_
                clip_grad_norm_(self.model.parameters(), self.clip_grad)
            self.optimizer.step()
        return loss
