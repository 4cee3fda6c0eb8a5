"""Flat, persistent buffers for the parameters that are not FP8 weights (embeddings, LayerNorms, biases), optionally
sharded over a data-parallel group like stock ZeRO shards them.

Replicated mode keeps parameters and optimizer states on every rank and all-reduces the gradients in one flat buffer
per dtype.  Sharded mode gives every tensor an owner rank: the flat buffers are laid out as ``world`` equal regions
(region r = the tensors owned by rank r), gradients are reduce-scattered so that each region's sum lands on its owner,
only the owner keeps optimizer states and updates, and the updated parameters are all-gathered region by region
(the reference leaves these parameters to DeepSpeed's own partitioning, msamp/deepspeed/runtime/zero/fp8_stage_1_and_2.py:36-68,
and to torch FSDP's flat parameters).
"""
import torch
import torch.distributed as dist

from msamp.common.utils.dist import DistUtil


def _pad16(n):
    return (n + 15) // 16 * 16


def partition_greedy(sizes, world):
    """Each tensor (in order) goes to the currently least-loaded rank; ties to the lowest rank (deterministic on every rank)."""
    load = [0] * world
    owners = []
    for n in sizes:
        r = min(range(world), key=lambda k: (load[k], k))
        owners.append(r)
        load[r] += n
    return owners


class HighPrecisionShards:
    """Gradient exchange (and, when ``shard`` is set, ownership) of a list of plain ``torch`` parameters."""
    def __init__(self, params, group=None, shard=True, device=None):
        self.params = list(params)
        self.group = group
        self.world = DistUtil.get_world_size(group)
        self.rank = DistUtil.get_rank(group)
        self.shard = bool(shard) and self.world > 1
        self.device = device if device is not None else (self.params[0].device if self.params else torch.device('cpu'))
        self.owner = [self.rank] * len(self.params)
        self.layout = {}    # dtype -> dict(region, params=[(index, offset)], flat_grad, flat_param or None)
        if self.world == 1 or not self.params:
            return
        if self.shard:
            self.owner = partition_greedy([p.numel() for p in self.params], self.world)
        by_dtype = {}
        for k, p in enumerate(self.params):
            by_dtype.setdefault(p.dtype, []).append(k)
        for dtype, idxs in by_dtype.items():
            fill = [0] * self.world
            place = []
            for k in idxs:
                r = self.owner[k] if self.shard else 0
                place.append((k, r, fill[r]))
                fill[r] += _pad16(self.params[k].numel())
            region = max(max(fill), 16) if self.shard else max(fill[0], 16)
            total = region * (self.world if self.shard else 1)
            flat_grad = torch.zeros(total, dtype=dtype, device=self.device)
            flat_param = None
            entries = [(k, r * region + off) for k, r, off in place]
            if self.shard:
                flat_param = torch.zeros(total, dtype=dtype, device=self.device)
                for k, off in entries:
                    p = self.params[k]
                    view = flat_param[off:off + p.numel()].view(p.shape)
                    view.copy_(p.data)
                    p.data = view
            self.layout[dtype] = dict(region=region, params=entries, flat_grad=flat_grad, flat_param=flat_param)

    def owned(self):
        """The parameters this rank updates (all of them when not sharded)."""
        return [p for k, p in enumerate(self.params) if self.owner[k] == self.rank]

    def bind_optimizer(self, optimizer):
        """Drop from ``optimizer`` the parameters (and states) of tensors another rank owns."""
        if not self.shard:
            return
        mine = {id(p) for p in self.owned()}
        ids = {id(p) for p in self.params}
        for group in optimizer.param_groups:
            group['params'] = [p for p in group['params'] if id(p) not in ids or id(p) in mine]
        for p in list(optimizer.state.keys()):
            if id(p) in ids and id(p) not in mine:
                del optimizer.state[p]

    def reduce_grads(self):
        """Average the gradients over the group; in sharded mode only the owner ends up with the result (``p.grad`` of
        every parameter becomes a view of the flat gradient buffer)."""
        if self.world == 1:
            return
        backend = dist.get_backend(self.group)
        for lay in self.layout.values():
            flat = lay['flat_grad']
            for k, off in lay['params']:
                p = self.params[k]
                view = flat[off:off + p.numel()].view(p.shape)
                if p.grad is not None and p.grad.data_ptr() != view.data_ptr():
                    view.copy_(p.grad)
                p.grad = view
            region = lay['region']
            if self.shard:
                mine = flat[self.rank * region:(self.rank + 1) * region]
                if backend == 'nccl':
                    dist.reduce_scatter_tensor(mine, flat, group=self.group)
                else:
                    dist.all_reduce(flat, group=self.group)
                mine.div_(self.world)
            else:
                dist.all_reduce(flat, group=self.group)
                flat.div_(self.world)

    def gather_params(self):
        """Publish the owners' updated parameters to every rank (sharded mode)."""
        if not self.shard:
            return
        backend = dist.get_backend(self.group)
        for lay in self.layout.values():
            flat, region = lay['flat_param'], lay['region']
            mine = flat[self.rank * region:(self.rank + 1) * region]
            if backend == 'nccl':
                dist.all_gather_into_tensor(flat, mine, group=self.group)
            else:
                parts = [torch.empty_like(mine) for _ in range(self.world)]
                dist.all_gather(parts, mine.clone(), group=self.group)
                for r, part in enumerate(parts):
                    if r != self.rank:
                        flat[r * region:(r + 1) * region].copy_(part)

    def clear_grads(self):
        for lay in self.layout.values():
            lay['flat_grad'].zero_()
        for p in self.params:
            p.grad = None
