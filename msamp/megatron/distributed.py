"""Local DDP for Megatron with FP8 main gradients (reference: msamp/megatron/distributed.py:17-216).

* High-precision parameters get ``main_grad`` views into one contiguous buffer per dtype.
* FP8Linear weights get ``main_grad`` ScalingTensors that live in one ``uint8`` buffer, laid out **by owning
  data-parallel rank** (greedy whole-tensor balance) with flat ``scale / scale_inv / amax`` arrays, so that
  the distributed optimizer can treat rank r's slice as its shard.
* Each weight's backward-post hook accumulates the fresh high-precision wgrad into that FP8 buffer with the
  fused ``add_to_fp8`` kernel (dequantise + add + new scale + requantise).
"""
import torch
import torch.distributed as dist

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingMeta, ScalingTensor
from msamp.megatron import parallel_state as mpu
from msamp.nn.parameter import ScalingParameter
from msamp.operators.arithmetic import Arithmetic
from msamp.parallel.zero import partition_tensors

E4M3 = Dtypes.kfloat8_e4m3


class MemoryBuffer:
    """Contiguous typed buffer handing out shaped views."""
    def __init__(self, numel, dtype, device):
        self.numel, self.dtype = numel, dtype
        self.data = torch.zeros(max(numel, 1), dtype=dtype, device=device)

    def zero(self):
        self.data.zero_()

    def get(self, shape, start):
        end = start + shape.numel()
        if end > self.numel:
            raise RuntimeError('requested tensor is out of the buffer range')
        return self.data[start:end].view(shape)


class FP8DistributedDataParallel(torch.nn.Module):
    """Gradient-buffer manager with the constructor of Megatron's local DDP.

    Args:
        module: model whose FP8 linears carry ScalingParameters.
        accumulate_allreduce_grads_in_fp32: keep high-precision main grads in fp32.
        use_contiguous_buffers: must be True (FP8 main grads need the flat layout).
    """
    def __init__(self, module, accumulate_allreduce_grads_in_fp32=True, use_contiguous_buffers=True):
        super().__init__()
        if not use_contiguous_buffers:
            raise ValueError('FP8DistributedDataParallel needs use_contiguous_buffers=True')
        self.module = module
        self.accumulate_allreduce_grads_in_fp32 = accumulate_allreduce_grads_in_fp32
        self.use_contiguous_buffers = True
        self.dp_group = mpu.get_data_parallel_group()
        self.dp_world = mpu.get_data_parallel_world_size()
        params = [p for p in module.parameters() if p.requires_grad]
        self.fp8_params = [p for p in params if isinstance(p, ScalingParameter)]
        self.hp_params = [p for p in params if not isinstance(p, ScalingParameter)]
        device = params[0].device
        # ---- high precision: one buffer per main-grad dtype
        self._grad_buffers = {}
        self._grad_buffer_param_index_map = {}
        sizes = {}
        for p in self.hp_params:
            dt = torch.float32 if accumulate_allreduce_grads_in_fp32 else p.dtype
            sizes[dt] = sizes.get(dt, 0) + p.numel()
        for dt, n in sizes.items():
            self._grad_buffers[dt] = MemoryBuffer(n, dt, device)
            self._grad_buffer_param_index_map[dt] = {}
        cursor = dict(sizes)
        for p in self.hp_params:
            dt = torch.float32 if accumulate_allreduce_grads_in_fp32 else p.dtype
            cursor[dt] -= p.numel()
            p.main_grad = self._grad_buffers[dt].get(p.shape, cursor[dt])
            self._grad_buffer_param_index_map[dt][p] = (cursor[dt], cursor[dt] + p.numel())
        # ---- FP8: one uint8 buffer ordered by owner rank, flat metas
        n = len(self.fp8_params)
        owners = partition_tensors([p.numel() for p in self.fp8_params], self.dp_world)
        self.fp8_owners = owners
        order = sorted(range(n), key=lambda i: (owners[i], i))
        total = sum(p.numel() for p in self.fp8_params)
        self._fp8_grad_buffer = MemoryBuffer(total, torch.uint8, device)
        self._grad_buffers[torch.uint8] = self._fp8_grad_buffer
        self._grad_buffer_param_index_map[torch.uint8] = {}
        self.fp8_partitions = [[0, 0] for _ in range(self.dp_world)]
        self.scales = torch.ones(max(n, 1), device=device)
        self.scale_invs = torch.ones(max(n, 1), device=device)
        self.amaxs = torch.zeros(max(n, 1), device=device)
        start = 0
        for slot, i in enumerate(order):
            p = self.fp8_params[i]
            meta = ScalingMeta(E4M3, scale=self.scales[slot], scale_inv=self.scale_invs[slot], amax=self.amaxs[slot:slot + 1], window_size=1)
            meta.pre_scale = 1.0 / self.dp_world
            p.main_grad = ScalingTensor(self._fp8_grad_buffer.get(p.shape, start), meta)
            self._grad_buffer_param_index_map[torch.uint8][p] = (start, start + p.numel())
            part = self.fp8_partitions[owners[i]]
            if part[1] == part[0]:
                part[0] = start
            part[1] = start + p.numel()
            start += p.numel()
        for r in range(self.dp_world):
            if self.fp8_partitions[r][1] == self.fp8_partitions[r][0]:
                self.fp8_partitions[r] = [start, start]
        # ---- hooks
        self._hooks = []
        for p in self.fp8_params:
            self._hooks.append(p.register_backward_post_hook(self._make_fp8_hook(p)))
        for p in self.hp_params:
            self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hp_hook()))

    @staticmethod
    def _make_fp8_hook(param):
        def hook(*unused):
            grad = param.grad
            if grad is None:
                return
            if isinstance(grad, ScalingTensor):
                grad = grad.float()
            mg = param.main_grad
            Arithmetic.add_to_fp8(mg.value.view(-1), mg.meta, grad.contiguous().view(-1))
            param.grad = None

        return hook

    @staticmethod
    def _make_hp_hook():
        def hook(param):
            if param.grad is not None:
                param.main_grad.add_(param.grad.to(param.main_grad.dtype))
                param.grad = None

        return hook

    def forward(self, *inputs, **kwargs):
        return self.module(*inputs, **kwargs)

    def state_dict(self, *args, **kwargs):
        return self.module.state_dict(*args, **kwargs)

    def load_state_dict(self, state_dict, strict=True):
        return self.module.load_state_dict(state_dict, strict=strict)

    def zero_grad_buffer(self):
        """Set every main-grad buffer to zero (call at the start of each training iteration)."""
        for buf in self._grad_buffers.values():
            buf.zero()

    def broadcast_params(self):
        """Make every data-parallel replica start from rank 0's parameters."""
        if self.dp_world == 1:
            return
        src = dist.get_global_rank(self.dp_group, 0) if self.dp_group is not None else 0
        for p in self.module.parameters():
            if isinstance(p, ScalingTensor):
                dist.broadcast(p.value, src=src, group=self.dp_group)
                dist.broadcast(p.meta.scale_inv, src=src, group=self.dp_group)
                dist.broadcast(p.meta.scale, src=src, group=self.dp_group)
                dist.broadcast(p.meta.amax, src=src, group=self.dp_group)
            else:
                dist.broadcast(p.data, src=src, group=self.dp_group)

    def allreduce_gradients(self):
        """Average all main grads over the data-parallel group (the distributed optimizer reduce-scatters instead)."""
        if self.dp_world == 1:
            return
        from msamp.common.tensor import TensorDist
        for dt, buf in self._grad_buffers.items():
            if dt == torch.uint8:
                continue
            buf.data.div_(self.dp_world)
            dist.all_reduce(buf.data, group=self.dp_group)
        # FP8: agree on the smallest scale, requantise where needed, then sum as FP8 numbers
        n = len(self.fp8_params)
        if n:
            agreed = self.scales[:n].clone()
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=self.dp_group)
            for p in self.fp8_params:
                mg = p.main_grad
                hp = mg.float()
                new_scale = torch.minimum(mg.meta.scale, agreed[(mg.meta.scale.data_ptr() - self.scales.data_ptr()) // 4])
                mg.meta.scale.copy_(new_scale)
                mg.value.copy_(hp.cast(E4M3, meta=_fixed_meta(new_scale)).value)
                mg.meta.scale_inv.copy_(torch.reciprocal(new_scale))
            TensorDist.all_reduce_avg([p.main_grad for p in self.fp8_params], group=self.dp_group)


def _fixed_meta(scale):
    """Meta that quantises with exactly ``scale`` (no in-time update)."""
    m = ScalingMeta(E4M3, scale=scale.clone(), window_size=2, device=scale.device)
    m.amax_counter += 2
    return m
