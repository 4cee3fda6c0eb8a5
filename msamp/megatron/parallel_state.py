"""Model-parallel process groups (a minimal ``mpu``).

Rank layout follows Megatron-LM: tensor-parallel ranks are adjacent, then data-parallel, then
pipeline stages, i.e. ``rank = pp_rank * (dp * tp) + dp_rank * tp + tp_rank``.  If Megatron-LM's
``megatron.core.parallel_state`` is importable and initialised, its groups are used instead.
"""
import torch.distributed as dist

_STATE = {'tp': None, 'dp': None, 'pp': None, 'mp': None, 'tp_size': 1, 'dp_size': 1, 'pp_size': 1, 'fused': None, 'init': False}


_CORE = [None, False]    # [megatron.core.parallel_state or None, import attempted]


def _core():
    """Megatron-LM's own parallel state when it is importable and initialised.  The import is attempted once: a failed
    import walks ``sys.path`` every time, and this function sits on the path of every tensor-parallel linear."""
    if not _CORE[1]:
        _CORE[1] = True
        try:
            from megatron.core import parallel_state as ps    # type: ignore
            _CORE[0] = ps
        except Exception:
            _CORE[0] = None
    ps = _CORE[0]
    if ps is not None:
        try:
            if ps.model_parallel_is_initialized():
                return ps
        except Exception:
            pass
    return None


def initialize_model_parallel(tensor_model_parallel_size=1, pipeline_model_parallel_size=1):
    """Create tensor-, data-, pipeline- and model-parallel groups for the current world."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    tp, pp = tensor_model_parallel_size, pipeline_model_parallel_size
    if world % (tp * pp):
        raise ValueError(f'world size {world} is not divisible by tp*pp = {tp * pp}')
    dp = world // (tp * pp)
    _STATE.update(tp_size=tp, dp_size=dp, pp_size=pp, init=True, fused=None)
    if world == 1:
        return
    for p in range(pp):
        for d in range(dp):
            ranks = [p * dp * tp + d * tp + t for t in range(tp)]
            g = dist.new_group(ranks)
            if rank in ranks:
                _STATE['tp'] = g
        for t in range(tp):
            ranks = [p * dp * tp + d * tp + t for d in range(dp)]
            g = dist.new_group(ranks)
            if rank in ranks:
                _STATE['dp'] = g
    for d in range(dp):
        for t in range(tp):
            ranks = [p * dp * tp + d * tp + t for p in range(pp)]
            g = dist.new_group(ranks)
            if rank in ranks:
                _STATE['pp'] = g
    for d in range(dp):
        ranks = [p * dp * tp + d * tp + t for p in range(pp) for t in range(tp)]
        g = dist.new_group(ranks)
        if rank in ranks:
            _STATE['mp'] = g


def destroy_model_parallel():
    fused = _STATE.get('fused')
    if fused is not None and hasattr(fused, 'close'):
        fused.close()    # frees the symmetric (IPC-shared) buffers of the fused GEMM kernels; collective over the group
    _STATE.update(tp=None, dp=None, pp=None, mp=None, tp_size=1, dp_size=1, pp_size=1, fused=None, init=False)


def model_parallel_is_initialized():
    return _STATE['init'] or _core() is not None


def get_tensor_model_parallel_group():
    c = _core()
    return c.get_tensor_model_parallel_group() if c else _STATE['tp']


def get_data_parallel_group():
    c = _core()
    return c.get_data_parallel_group() if c else _STATE['dp']


def get_pipeline_model_parallel_group():
    c = _core()
    return c.get_pipeline_model_parallel_group() if c else _STATE['pp']


def get_model_parallel_group():
    c = _core()
    return c.get_model_parallel_group() if c else _STATE['mp']


def get_tensor_model_parallel_world_size():
    c = _core()
    return c.get_tensor_model_parallel_world_size() if c else _STATE['tp_size']


def get_tensor_model_parallel_rank():
    c = _core()
    if c:
        return c.get_tensor_model_parallel_rank()
    g = _STATE['tp']
    return dist.get_rank(g) if g is not None else 0


def get_tensor_model_parallel_src_rank():
    """Global rank of the first member of this rank's tensor-parallel group."""
    c = _core()
    if c:
        return c.get_tensor_model_parallel_src_rank()
    rank = dist.get_rank() if dist.is_initialized() else 0
    return rank - get_tensor_model_parallel_rank()


def get_data_parallel_world_size():
    c = _core()
    return c.get_data_parallel_world_size() if c else _STATE['dp_size']


def get_data_parallel_rank():
    c = _core()
    if c:
        return c.get_data_parallel_rank()
    g = _STATE['dp']
    return dist.get_rank(g) if g is not None else 0


def get_fused_context(shard_bytes=0, out_bytes=0):
    """FusedGemmContext of the tensor-parallel group, created (or enlarged) collectively on first need."""
    from msamp.parallel.fused import FusedGemmContext
    ctx = _STATE['fused']
    if ctx is None or ctx.max_shard_bytes < shard_bytes or ctx.max_out_bytes < out_bytes:
        old_s = ctx.max_shard_bytes if ctx else 0
        old_o = ctx.max_out_bytes if ctx else 0
        ctx = FusedGemmContext(get_tensor_model_parallel_group(), max(shard_bytes, old_s), max(out_bytes, old_o))
        _STATE['fused'] = ctx
    return ctx
