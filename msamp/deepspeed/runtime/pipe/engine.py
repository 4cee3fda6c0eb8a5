"""Pipeline parallelism: stage partitioning and the 1F1B schedule over NCCL/gloo point-to-point.

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
        self._mp_group = None
        if dist.is_initialized() and world > 1:
            for s in range(num_stages):
                ranks = list(range(s * self.dp_size, (s + 1) * self.dp_size))
                g = dist.new_group(ranks)
                if rank in ranks:
                    self._dp_group = g
            for d in range(self.dp_size):
                ranks = [s * self.dp_size + d for s in range(num_stages)]    # one replica of the whole model
                g = dist.new_group(ranks)
                if rank in ranks:
                    self._mp_group = g

    def get_data_parallel_group(self):
        return self._dp_group

    def get_data_parallel_world_size(self):
        return self.dp_size

    def get_model_parallel_group(self):
        """The stages of this rank's model replica (gradient norms and overflow flags are combined over it)."""
        return self._mp_group

    def get_pipe_parallel_group(self):
        return self._mp_group

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
    """``train_batch(data_iter)`` runs the micro-batches of one step through the stages with the 1F1B schedule
    (warm-up forwards, then one forward and one backward alternately, then the remaining backwards), so a stage
    holds at most ``num_stages - stage_id`` activations, and ends with one optimizer step.

    Transfers between neighbours are posted as batched ``isend`` / ``irecv`` pairs (a send and a receive in
    opposite directions are always in one batch, which is what NCCL needs to make progress).  The shape of the
    activation is announced once, with the first tensor a stage sends; gradients have the shape of what was sent.
    """
    def __init__(self, *args, model=None, **kwargs):
        kwargs['mpu'] = kwargs.get('mpu') or model
        super().__init__(*args, model=model, **kwargs)
        self.__dict__['pipe'] = model    # the PipelineModule (also reachable as self.module); kept out of the submodule registry
        self._in_shape = None       # shape of the activation received from the previous stage
        self._meta_sent = False

    # ------------------------------------------------------------------ point-to-point helpers
    def _announce(self, t, dst):
        if not self._meta_sent:
            meta = torch.tensor([t.dim()] + list(t.shape) + [0] * (7 - t.dim()), dtype=torch.int64, device=t.device if t.is_cuda else 'cpu')
            dist.send(meta, dst)
            self._meta_sent = True

    def _learn_shape(self, src, device):
        if self._in_shape is None:
            meta = torch.zeros(8, dtype=torch.int64, device=device if device.type == 'cuda' else 'cpu')
            dist.recv(meta, src)
            self._in_shape = [int(v) for v in meta[1:1 + int(meta[0])]]

    @staticmethod
    def _exchange(send=None, dst=None, recv=None, src=None):
        """Post the given send and / or receive together and wait for both."""
        ops = []
        if send is not None:
            ops.append(dist.P2POp(dist.isend, send.contiguous(), dst))
        if recv is not None:
            ops.append(dist.P2POp(dist.irecv, recv, src))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        return recv

    def train_batch(self, data_iter=None):
        pipe = self.pipe if isinstance(self.pipe, PipelineModule) else self.module
        ga = self.gradient_accumulation_steps()
        device = next(p for p in self.module.parameters() if torch.is_tensor(p)).device
        act_dtype = getattr(self, 'activation_dtype', torch.float32)
        first, last = pipe.is_first_stage, pipe.is_last_stage
        warmup = min(pipe.num_stages - pipe.stage_id - 1, ga)
        steady = ga - warmup
        pending = []    # (input, output) of micro-batches whose backward has not run yet, oldest first
        losses = []

        def next_input(batch):
            if first:
                return batch[0].to(device)
            self._learn_shape(pipe.prev_rank, device)
            return torch.empty(self._in_shape, dtype=act_dtype, device=device)

        def forward(x, batch):
            if not first:
                x.requires_grad_()
            y = self.module(x)
            if last:
                y = pipe.loss_fn(y, batch[1].to(device)) / ga
                losses.append(y.detach())
            pending.append((x, y))
            return y

        def backward(grad):
            x, y = pending.pop(0)
            if last:
                scale = self.optimizer.cur_scale if hasattr(self.optimizer, 'cur_scale') else 1.0
                (y.float() * scale).backward()
            else:
                y.backward(grad)
            return None if first else x.grad

        def fetch():
            return next(data_iter) if (first or last) and data_iter is not None else None

        # warm-up: forwards only
        for _ in range(warmup):
            batch = fetch()
            x = next_input(batch)
            if not first:
                self._exchange(recv=x, src=pipe.prev_rank)
            y = forward(x, batch)
            if not last:
                self._announce(y, pipe.next_rank)
                self._exchange(send=y.detach(), dst=pipe.next_rank)
        # steady state: one forward, one backward
        batch = x = None
        if steady > 0:
            batch = fetch()
            x = next_input(batch)
            if not first:
                self._exchange(recv=x, src=pipe.prev_rank)
        for i in range(steady):
            y = forward(x, batch)
            grad = None
            if not last:
                self._announce(y, pipe.next_rank)
                grad = torch.empty_like(y)
                self._exchange(send=y.detach(), dst=pipe.next_rank, recv=grad, src=pipe.next_rank)
            dx = backward(grad)
            more = i + 1 < steady
            if more:
                batch = fetch()
                x = next_input(batch)
            if not first:
                self._exchange(send=dx, dst=pipe.prev_rank, recv=x if more else None, src=pipe.prev_rank)
        # cool-down: the remaining backwards
        for _ in range(warmup):
            grad = None
            if not last:
                grad = torch.empty_like(pending[0][1])
                self._exchange(recv=grad, src=pipe.next_rank)
            dx = backward(grad)
            if not first:
                self._exchange(send=dx, dst=pipe.prev_rank)
        self.micro_steps += ga - 1
        self.step()
        return torch.stack([l.float() for l in losses]).sum() if losses else torch.zeros((), device=device)
