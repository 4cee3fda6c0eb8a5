"""FP8 distributed optimizer with Megatron's interface (reference: msamp/megatron/optimizer/distrib_optimizer.py:20-1019).

Semantics kept from the reference: optimizer states and scaled-fp16 master weights of FP8 parameters
exist only on the owning data-parallel rank (whole-tensor ownership); model weights are e4m3;
``reduce_model_grads`` leaves each owner with the averaged FP8 gradients of its tensors;
``gather_model_params`` re-quantises the updated masters and distributes weights and ``scale_inv``;
``state_dict`` carries param groups and the grad scaler, the tensors go to a separate parameter-state
file as fp32 world buffers keyed by dtype (``torch.float32`` / ``torch.uint8``).

The data movement is delegated to ``msamp.parallel.zero.ZeroShardedOptimizer``: one fused NVLink kernel for
the gradient reduce-scatter (replacing the MIN-scale all-reduce + requantise + NCCL reduce-scatter), one for
cast + weight/scale broadcast.
"""
import torch
import torch.distributed as dist

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingTensor
from msamp.megatron import parallel_state as mpu
from msamp.megatron.optimizer.clip_grads import clip_grad_norm_fp32
from msamp.parallel.zero import ZeroShardedOptimizer


class FP8DistributedOptimizer:
    """Sharded optimizer for models wrapped by ``msamp.megatron.FP8DistributedDataParallel``."""
    def __init__(self, optimizer, clip_grad=0.0, log_num_zeros_in_grad=False, params_have_main_grad=True,
                 use_contiguous_buffers_in_local_ddp=True, fp16=False, bf16=True, params_dtype=torch.bfloat16, grad_scaler=None,
                 models=None):
        if not models:
            raise ValueError('FP8DistributedOptimizer needs the list of model chunks')
        if not use_contiguous_buffers_in_local_ddp:
            raise ValueError('the distributed optimizer needs contiguous gradient buffers')
        self.optimizer = optimizer
        self.clip_grad = clip_grad
        self.log_num_zeros_in_grad = log_num_zeros_in_grad
        self.params_have_main_grad = params_have_main_grad
        self.fp16, self.bf16, self.params_dtype = fp16, bf16, params_dtype
        self.grad_scaler = grad_scaler
        self.models = list(models)
        self.dp_group = mpu.get_data_parallel_group()
        holder = torch.nn.ModuleList([getattr(m, 'module', m) for m in self.models])
        self.zero = ZeroShardedOptimizer(holder, optimizer, stage=1, group=self.dp_group)
        # FP8 main grads now live in the sharded optimizer's (symmetric) flat buffer
        for p in self.zero.fp8_params:
            p.main_grad = ScalingTensor(p._grad_out, p._scaling_metas['wgrad'])
            p._grad_out = None    # megatron layers deliver high-precision wgrads to the DDP hook, which accumulates into main_grad
        self._found_inf = torch.zeros((), device=self.zero.device)

    # ------------------------------------------------------------------ Megatron optimizer interface
    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def zero_grad(self, set_to_none=True):
        for m in self.models:
            if hasattr(m, 'zero_grad_buffer'):
                m.zero_grad_buffer()
        for p in self.zero.fp8_params:
            p.grad = None
            p.main_grad.value.zero_()
        for p in self.zero.hp_params:
            p.grad = None
        if self.zero.hp_layout:
            self.zero._clear_hp_grads()

    def get_loss_scale(self):
        if self.grad_scaler is None:
            return torch.ones((), device=self.zero.device)
        return self.grad_scaler.scale

    def scale_loss(self, loss):
        return self.get_loss_scale() * loss

    def reduce_model_grads(self, args=None, timers=None):
        """Average gradients over the data-parallel group; FP8 gradients end up on their owners only."""
        for p in self.zero.hp_params:
            mg = getattr(p, 'main_grad', None)
            if mg is not None:
                p.grad = mg if mg.dtype == p.dtype else mg.to(p.dtype)
        for p in self.zero.fp8_params:
            p.grad = p.main_grad
        self.zero._reduce_fp8_grads()
        self.zero._reduce_hp_grads()

    def gather_model_params(self, args=None, timers=None):
        """Publish the updated weights (and their ``scale_inv``) of every owner to all data-parallel ranks."""
        self.zero._publish_weights()
        self.zero._gather_hp_params()

    def _hp_updated_here(self):
        """High-precision parameters this rank updates: all of them on one data-parallel rank, else the ones it owns
        (the sharded optimizer partitions them over the data-parallel group like the FP8 weights)."""
        return self.zero._owned_hp() if (self.zero.sharded and self.zero.world > 1) else self.zero.hp_params

    def _unscale_and_check(self):
        if self.grad_scaler is None:
            return False
        inv = torch.reciprocal(self.grad_scaler.scale).reshape(1)
        self._found_inf.zero_()
        grads = [m.grad for m in self.zero.masters.values() if m.grad is not None] + [p.grad for p in self._hp_updated_here() if p.grad is not None]
        torch._amp_foreach_non_finite_check_and_unscale_(grads, self._found_inf.reshape(1), inv)
        dist.all_reduce(self._found_inf, op=dist.ReduceOp.MAX, group=mpu.get_model_parallel_group()) if dist.is_initialized() else None
        return bool(self._found_inf.item() > 0)

    @torch.no_grad()
    def step(self, args=None, timers=None):
        """Returns ``(update_successful, grad_norm, num_zeros_in_grad)`` like Megatron's mixed-precision optimizers."""
        for i, m in self.zero.masters.items():
            m.grad = self.zero.fp8_params[i].grad
        found_inf = self._unscale_and_check()
        if self.grad_scaler is not None:
            self.grad_scaler.update(found_inf)
        if found_inf:
            return False, None, None
        grad_norm = None
        if self.clip_grad > 0.0:
            hp_here = self._hp_updated_here()
            params = list(self.zero.masters.values()) + hp_here
            grads_for_norm = [m.grad for m in self.zero.masters.values() if m.grad is not None]
            tp_rank = mpu.get_tensor_model_parallel_rank()
            dp_rank = mpu.get_data_parallel_rank()
            owner_counts = self.zero.sharded and self.zero.world > 1
            for p in hp_here:
                if p.grad is None:
                    continue
                is_tp = getattr(p, 'tensor_model_parallel', False)
                if (owner_counts or dp_rank == 0) and (is_tp or tp_rank == 0):    # replicated params count once
                    grads_for_norm.append(p.grad)
            # Every gradient is counted on exactly one rank of the whole job (FP8 and high-precision gradients on their
            # owner inside the data-parallel group, tensor-parallel replicas on tensor-parallel rank 0), so the norm is
            # summed over all ranks: data-parallel replicas must agree on the clip coefficient.
            group = dist.group.WORLD if dist.is_initialized() and dist.get_world_size() > 1 else None
            grad_norm = clip_grad_norm_fp32(params, grads_for_norm, self.clip_grad, 2, model_parallel_group=group)
        self.optimizer.step()
        self.gather_model_params(args, timers)
        for m in self.zero.masters.values():
            m.grad = None
        return True, grad_norm, None

    # ------------------------------------------------------------------ checkpoint
    def state_dict(self):
        """Param groups (with ``step``, without tensors) and the grad scaler; tensors go to ``save_parameter_state``."""
        inner = self.optimizer.state_dict()
        groups = []
        steps = [s.get('step', 0) for s in inner['state'].values()]
        for g in inner['param_groups']:
            g = {k: v for k, v in g.items() if k != 'params'}
            g['step'] = max(steps) if steps else 0
            groups.append(g)
        sd = {'optimizer': {'param_groups': groups}}
        if self.grad_scaler is not None:
            sd['grad_scaler'] = self.grad_scaler.state_dict()
        return sd

    def load_state_dict(self, state_dict):
        for g, saved in zip(self.optimizer.param_groups, state_dict['optimizer']['param_groups']):
            for k, v in saved.items():
                if k not in ('params', 'step'):
                    g[k] = v
            self._restored_step = saved.get('step', 0)
        if self.grad_scaler is not None and 'grad_scaler' in state_dict:
            self.grad_scaler.load_state_dict(state_dict['grad_scaler'])

    def _gather_world(self, payload):
        """Collect every data-parallel rank's (CPU) piece; the reference moves the same data through a gloo group."""
        world = mpu.get_data_parallel_world_size()
        if world == 1:
            return [payload]
        pieces = [None] * world
        dist.all_gather_object(pieces, payload, group=self.dp_group)
        return pieces

    def save_parameter_state(self, filename):
        """Write master weights and Adam moments as fp32 buffers: ``state[model_idx][dtype] = {'param','exp_avg','exp_avg_sq'}``."""
        z = self.zero
        local = {}
        for i, m in z.masters.items():
            st = self.optimizer.state.get(m, {})
            local[i] = {
                'param': m.float().cpu(),
                'exp_avg': st['exp_avg'].float().cpu() if 'exp_avg' in st else torch.zeros(m.shape),
                'exp_avg_sq': st['exp_avg_sq'].float().cpu() if 'exp_avg_sq' in st else torch.zeros(m.shape),
                'step': st.get('step', 0),
            }
        hp = {}
        for j, p in enumerate(z.hp_params):
            if z.hp_owner[j] != z.rank:
                continue    # states of a sharded high-precision parameter live on its owner
            st = self.optimizer.state.get(p, {})
            hp[j] = {
                'param': p.detach().float().cpu(),
                'exp_avg': st['exp_avg'].float().cpu() if 'exp_avg' in st else torch.zeros(p.shape),
                'exp_avg_sq': st['exp_avg_sq'].float().cpu() if 'exp_avg_sq' in st else torch.zeros(p.shape),
                'step': st.get('step', 0),
            }
        pieces = self._gather_world({'fp8': local, 'hp': hp})
        if mpu.get_data_parallel_rank() == 0:
            merged = {}
            hp = {}
            for piece in pieces:
                merged.update(piece['fp8'])
                hp.update(piece['hp'])
            order = sorted(merged)
            state = {0: {
                torch.uint8: {k: torch.cat([merged[i][k].reshape(-1) for i in order]) if order else torch.zeros(0) for k in ('param', 'exp_avg', 'exp_avg_sq')},
                torch.float32: {k: torch.cat([hp[j][k].reshape(-1) for j in sorted(hp)]) if hp else torch.zeros(0) for k in ('param', 'exp_avg', 'exp_avg_sq')},
            }, 'steps': {'fp8': {i: merged[i]['step'] for i in order}, 'hp': {j: hp[j]['step'] for j in hp}}}
            torch.save(state, filename)

    def load_parameter_state(self, filename):
        """Inverse of ``save_parameter_state``: every rank reads the file and keeps (re-quantises) what it owns."""
        z = self.zero
        state = torch.load(filename, map_location='cpu', weights_only=False)
        bufs = state[0]
        off = 0
        for i, p in enumerate(z.fp8_params):
            n = p.numel()
            if i in z.masters:
                m = z.masters[i]
                w = bufs[torch.uint8]['param'][off:off + n].view(p.shape).to(z.device)
                m.copy_(w.cast(Dtypes.kfloat16))
                st = self.optimizer.state[m]
                st['step'] = state['steps']['fp8'].get(i, 0)
                ea = bufs[torch.uint8]['exp_avg'][off:off + n].view(p.shape).to(z.device)
                es = bufs[torch.uint8]['exp_avg_sq'][off:off + n].view(p.shape).to(z.device)
                st['exp_avg'] = self.optimizer._get_state_tensor(ea, self.optimizer.exp_avg_dtype)
                st['exp_avg_sq'] = self.optimizer._get_state_tensor(es, self.optimizer.exp_avg_sq_dtype)
            off += n
        off = 0
        for j, p in enumerate(z.hp_params):
            n = p.numel()
            p.data.copy_(bufs[torch.float32]['param'][off:off + n].view(p.shape).to(p.dtype))
            if z.hp_owner[j] != z.rank:
                off += n
                continue
            st = self.optimizer.state[p]
            st['step'] = state['steps']['hp'].get(j, 0)
            st['exp_avg'] = self.optimizer._get_state_tensor(bufs[torch.float32]['exp_avg'][off:off + n].view(p.shape).to(z.device), self.optimizer.exp_avg_dtype)
            st['exp_avg_sq'] = self.optimizer._get_state_tensor(bufs[torch.float32]['exp_avg_sq'][off:off + n].view(p.shape).to(z.device), self.optimizer.exp_avg_sq_dtype)
            off += n
        self.gather_model_params()
