"""Pipeline parallelism: stage partitioning and a GPipe-style schedule over NCCL/gloo point-to-point.

Activations and their gradients travel between adjacent stages in high precision with
``torch.distributed`` send/recv (the reference inherits exactly this from DeepSpeed and adds only the
gradient-reduction hooks for ZeRO / BF16, msamp/deepspeed/runtime/pipe/engine.py:14-48); FP8 is used
inside each stage's linears and for the data-parallel gradient exchange of the stage's optimizer.
"""
import torch
import torch.distributed as dist

from msamp.deepspeed.runtime.engine import MSAMPDeepSpeedEngine


class PipelineModule(torch.nn.Module):
    """A model given as a list of layers; each pipeline rank keeps a contiguous slice.

    Args:
        layers: list of ``nn.Module`` (or callables building one).
        num_stages: pipeline depth.  stage_id: this rank's stage (default: ``rank % num_stages`` ... derived from the world).
        loss_fn: ``loss_fn(output, labels)`` evaluated on the last stage.
    """
    def __init__(self, layers, num_stages, loss_fn=None, stage_id=None, partition_method='uniform'):
        super().__init__()
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        if world % num_stages:
            raise ValueError('world size must be divisible by num_stages')
        self.num_stages = num_stages
        self.dp_size = world // num_stages
        self.stage_id = stage_id if stage_id is not None else rank // self.dp_size
        self.loss_fn = loss_fn
        n = len(layers)
        per = [n // num_stages + (1 if i < n % num_stages else 0) for i in range(num_stages)]
        start = sum(per[:self.stage_id])
        mine = layers[start:start + per[self.stage_id]]
        self.layers = torch.nn.ModuleList([l() if not isinstance(l, torch.nn.Module) and callable(l) else l for l in mine])
        self.prev_rank = rank - self.dp_size if self.stage_id > 0 else None
        self.next_rank = rank + self.dp_size if self.stage_id < num_stages - 1 else None
        self._dp_group = None
        if dist.is_initialized() and world > 1:
            for s in range(num_stages):
                ranks = list(range(s * self.dp_size, (s + 1) * self.dp_size))
                g = dist.new_group(ranks)
                if rank in ranks:
                    self._dp_group = g

    def get_data_parallel_group(self):
        return self._dp_group

    def get_data_parallel_world_size(self):
        return self.dp_size

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return x

    @property
    def is_first_stage(self):
        return self.stage_id == 0

    @property
    def is_last_stage(self):
        return self.stage_id == self.num_stages - 1


class MSAMPPipelineEngine(MSAMPDeepSpeedEngine):
    """``train_batch(data_iter)`` runs all micro-batches forward, then backward in reverse order, then one optimizer step."""
    def __init__(self, *args, model=None, **kwargs):
        kwargs['mpu'] = kwargs.get('mpu') or model
        super().__init__(*args, model=model, **kwargs)
        self.__dict__['pipe'] = model    # the PipelineModule (also reachable as self.module); kept out of the submodule registry

    def _send(self, t, dst):
        meta = torch.tensor([t.dim()] + list(t.shape) + [0] * (7 - t.dim()), dtype=torch.int64, device=t.device if t.is_cuda else 'cpu')
        dist.send(meta, dst)
        dist.send(t.contiguous(), dst)

    def _recv(self, src, dtype, device):
        meta = torch.zeros(8, dtype=torch.int64, device=device if device.type == 'cuda' else 'cpu')
        dist.recv(meta, src)
        shape = [int(v) for v in meta[1:1 + int(meta[0])]]
        t = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(t, src)
        return t

    def train_batch(self, data_iter=None):
        pipe = self.pipe if isinstance(self.pipe, PipelineModule) else self.module
        ga = self.gradient_accumulation_steps()
        device = next(p for p in self.module.parameters() if torch.is_tensor(p)).device
        act_dtype = getattr(self, 'activation_dtype', torch.float32)
        inputs, outputs, losses = [], [], []
        for _ in range(ga):
            batch = next(data_iter) if (pipe.is_first_stage or pipe.is_last_stage) and data_iter is not None else None
            if pipe.is_first_stage:
                x = batch[0].to(device)
            else:
                x = self._recv(pipe.prev_rank, act_dtype, device).requires_grad_()
            y = self.module(x)
            inputs.append(x)
            if pipe.is_last_stage:
                loss = pipe.loss_fn(y, batch[1].to(device)) / ga
                losses.append(loss)
                outputs.append(loss)
            else:
                self._send(y.detach(), pipe.next_rank)
                outputs.append(y)
        for i in reversed(range(ga)):
            if pipe.is_last_stage:
                scale = self.optimizer.cur_scale if hasattr(self.optimizer, 'cur_scale') else 1.0
                (outputs[i].float() * scale).backward()
            else:
                g = self._recv(pipe.next_rank, outputs[i].dtype, device)
                outputs[i].backward(g)
            if not pipe.is_first_stage:
                self._send(inputs[i].grad, pipe.prev_rank)
        self.micro_steps += ga - 1
        self.step()
        total = torch.stack([l.detach().float() for l in losses]).sum() if losses else torch.zeros((), device=device)
        if dist.is_initialized() and dist.get_world_size() > 1:
            last = (pipe.num_stages - 1) * pipe.dp_size
            dist.broadcast(total, src=last + (dist.get_rank() % pipe.dp_size) if pipe.dp_size > 1 else last) if pipe.dp_size == 1 else None
        return total
