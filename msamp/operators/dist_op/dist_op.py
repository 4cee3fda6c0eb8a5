"""Collectives on FP8 payloads.

The reference obtains FP8 reductions by preloading a shim that rewrites the NCCL datatype of
uint8 buffers while a process-global flag is set (msamp/operators/dist_op/dist_op.py:13-87,
dist.cpp:39-104).  NCCL >= 2.24 has native ``float8`` datatypes, so here a byte buffer is simply
viewed as ``torch.float8_e4m3fn`` / ``torch.float8_e5m2`` for the call – no global state, safe with
async ops.  On backends without FP8 arithmetic (gloo, used by the CPU tests) the reduction is
emulated: gather the bytes, reduce in fp32, round once with saturation.
``enable_fp8`` / ``disable_fp8`` are kept as a thread-local context for API compatibility.
"""
import threading

import torch
import torch.distributed as dist

from msamp.common.dtype import Dtypes, Floating

_F8 = Dtypes.qtype_to_float8
_state = threading.local()


class _Done:
    """Completed-work handle returned by emulated async collectives."""
    def wait(self):
        return True

    def is_completed(self):
        return True


def _emulated_reduce(tensor, qtype, op, group, dst=None):
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    parts = [torch.empty_like(tensor) for _ in range(world)]
    dist.all_gather(parts, tensor.contiguous(), group=group)
    vals = torch.stack([p.view(torch.uint8).view(_F8[qtype]).float() for p in parts])
    if op == dist.ReduceOp.SUM:
        red = vals.sum(0)
    elif op == dist.ReduceOp.MAX:
        red = vals.max(0).values
    elif op == dist.ReduceOp.MIN:
        red = vals.min(0).values
    elif op == dist.ReduceOp.AVG:
        red = vals.mean(0)
    else:
        raise ValueError(f'unsupported reduce op {op}')
    fmax = Floating.qfp_max[qtype]
    red = torch.where(torch.isnan(red), red, red.clamp(-fmax, fmax))
    me = dist.get_global_rank(group, rank) if group is not None else rank
    if dst is None or me == dst:
        tensor.copy_(red.to(_F8[qtype]).view(tensor.dtype).view_as(tensor))


class DistOp:
    """All-reduce / reduce / reduce-scatter / all-gather for high-precision and FP8 buffers."""
    @staticmethod
    def enable_fp8(qtype):
        if not Dtypes.is_fp8_qtype(qtype):
            raise RuntimeError(f'qtype {qtype} is not supported in enable_fp8.')
        _state.qtype = qtype

    @staticmethod
    def disable_fp8():
        _state.qtype = None

    @staticmethod
    def _native_fp8(tensor, group):
        return tensor.is_cuda and dist.get_backend(group) == 'nccl'

    @classmethod
    def all_reduce(cls, tensor, qtype, op=dist.ReduceOp.SUM, group=None, async_op=False):
        if Dtypes.is_fp8_qtype(qtype):
            if cls._native_fp8(tensor, group):
                return dist.all_reduce(tensor.view(_F8[qtype]), op=op, group=group, async_op=async_op)
            _emulated_reduce(tensor, qtype, op, group)
            return _Done() if async_op else None
        return dist.all_reduce(tensor, op=op, group=group, async_op=async_op)

    @classmethod
    def reduce(cls, tensor, qtype, dst, op=dist.ReduceOp.SUM, group=None, async_op=False):
        if Dtypes.is_fp8_qtype(qtype):
            if cls._native_fp8(tensor, group):
                return dist.reduce(tensor.view(_F8[qtype]), dst=dst, op=op, group=group, async_op=async_op)
            _emulated_reduce(tensor, qtype, op, group, dst=dst)
            return _Done() if async_op else None
        return dist.reduce(tensor, dst=dst, op=op, group=group, async_op=async_op)

    @classmethod
    def reduce_scatter(cls, output, input, qtype, op=dist.ReduceOp.SUM, group=None, async_op=False):
        """``output`` receives this rank's slice of the reduction of ``input`` (flat, world * len(output))."""
        if Dtypes.is_fp8_qtype(qtype):
            if cls._native_fp8(input, group):
                return dist.reduce_scatter_tensor(output.view(_F8[qtype]), input.view(_F8[qtype]), op=op, group=group, async_op=async_op)
            tmp = input.clone()
            _emulated_reduce(tmp, qtype, op, group)
            n = output.numel()
            r = dist.get_rank(group)
            output.copy_(tmp.view(-1)[r * n:(r + 1) * n].view_as(output))
            return _Done() if async_op else None
        if dist.get_backend(group) == 'nccl':
            return dist.reduce_scatter_tensor(output, input, op=op, group=group, async_op=async_op)
        tmp = input.clone()
        dist.all_reduce(tmp, op=op, group=group)
        n = output.numel()
        r = dist.get_rank(group)
        output.copy_(tmp.view(-1)[r * n:(r + 1) * n].view_as(output))
        return _Done() if async_op else None
