"""Bucketed collectives over lists of Tensor / ScalingTensor.

Tensors are packed into one flat buffer per bucket, the collective runs once per bucket, and the
results are copied back in place.  Bucket sizes are counted in **elements**, as the reference
actually does (msamp/common/tensor/tensor_dist.py:17-18, 58-59).
"""
import torch
import torch.distributed as dist

from msamp.common.dtype import Dtypes
from msamp.common.utils.dist import DistUtil
from msamp.common.tensor.tensor import ScalingTensor


class TensorDist:
    """Broadcast / all-reduce helpers for mixed lists of plain and scaling tensors."""
    BROADCAST_BUCKET_SIZE = 512 * (1024**2)
    ALL_REDUCE_BUCKET_SIZE = 512 * (1024**2)

    @staticmethod
    def _flush(bucket, dist_fn):
        if not bucket:
            return
        if len(bucket) == 1 and bucket[0].is_contiguous():
            dist_fn(bucket[0].view(-1))
            return
        flat = torch.cat([t.reshape(-1) for t in bucket])
        dist_fn(flat)
        off = 0
        for t in bucket:
            n = t.numel()
            t.copy_(flat[off:off + n].view_as(t))
            off += n

    @classmethod
    def _dist_tensors_by_bucket(cls, tensors, dist_fn, bucket_size, group=None):
        if DistUtil.get_world_size(group) == 1:
            return
        if not isinstance(tensors, (list, tuple)):
            tensors = [tensors]
        bucket, n = [], 0
        for t in tensors:
            if t is None:
                continue
            if isinstance(t, ScalingTensor):
                t = t.value
            bucket.append(t)
            n += t.numel()
            if n >= bucket_size:
                cls._flush(bucket, dist_fn)
                bucket, n = [], 0
        cls._flush(bucket, dist_fn)

    @classmethod
    def broadcast(cls, tensors, src, bucket_size=BROADCAST_BUCKET_SIZE, group=None):
        """Broadcast values (and, for ScalingTensors, their ``scale_inv``) from ``src``."""
        if DistUtil.get_world_size(group) == 1 or len(tensors) == 0:
            return

        def dist_fn(x):
            dist.broadcast(x, src=src, group=group)

        if isinstance(tensors[0], ScalingTensor):
            cls._dist_tensors_by_bucket([p.value for p in tensors], dist_fn, bucket_size, group)
            cls._dist_tensors_by_bucket([p.meta.scale_inv for p in tensors], dist_fn, bucket_size, group)
            cls._dist_tensors_by_bucket([p.meta.scale for p in tensors], dist_fn, bucket_size, group)
        else:
            cls._dist_tensors_by_bucket(tensors, dist_fn, bucket_size, group)

    @classmethod
    def all_reduce(cls, tensors, op, bucket_size=ALL_REDUCE_BUCKET_SIZE, group=None):
        """All-reduce tensors of one common qtype; FP8 payloads are reduced as FP8 numbers, not bytes."""
        from msamp.operators.dist_op import DistOp
        if len(tensors) == 0:
            return
        qtype = tensors[0].qtype
        if not all(qtype == t.qtype for t in tensors):
            raise TypeError('all_reduce only supports tensors with same qtype')

        def dist_fn(x):
            DistOp.all_reduce(x, qtype, op, group=group)

        cls._dist_tensors_by_bucket(tensors, dist_fn, bucket_size, group)

    @classmethod
    def all_reduce_avg(cls, tensors, bucket_size=ALL_REDUCE_BUCKET_SIZE, group=None):
        """Average over ranks. FP8 tensors are summed and their ``scale_inv`` divided by the world size."""
        world = DistUtil.get_world_size(group)
        if world == 1 or len(tensors) == 0:
            return
        if Dtypes.is_fp8_qtype(tensors[0].qtype):
            first = tensors[0].value if isinstance(tensors[0], ScalingTensor) else tensors[0]
            if first.is_cuda and DistUtil.backend(group) == 'nccl':
                # NCCL sums the FP8 numbers; the division goes into scale_inv (the reference's rule).
                cls.all_reduce(tensors, dist.ReduceOp.SUM, bucket_size, group=group)
                for t in tensors:
                    t.div_(world)
            else:
                # emulated collective: the mean is formed in fp32 and rounded once, so it cannot saturate
                cls.all_reduce(tensors, dist.ReduceOp.AVG, bucket_size, group=group)
        else:
            op = dist.ReduceOp.AVG if DistUtil.backend(group) == 'nccl' else dist.ReduceOp.SUM
            cls.all_reduce(tensors, op, bucket_size, group=group)
            if op == dist.ReduceOp.SUM:
                for t in tensors:
                    (t.value if isinstance(t, ScalingTensor) else t).div_(world)

    @classmethod
    def all_reduce_sum(cls, tensors, bucket_size=ALL_REDUCE_BUCKET_SIZE, group=None):
        if DistUtil.get_world_size(group) == 1 or len(tensors) == 0:
            return
        cls.all_reduce(tensors, dist.ReduceOp.SUM, bucket_size, group=group)
