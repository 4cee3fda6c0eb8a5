"""GPT decoder with Megatron-style tensor parallelism and sequence parallelism on msamp's fused kernels.

Inside a tensor-parallel group of size ``tp`` every rank holds ``1/tp`` of each projection
(``ColumnParallelLinear`` for QKV / FC1 / LM head, ``RowParallelLinear`` for the attention output and
FC2) and ``1/tp`` of the tokens wherever the computation is token-wise (embeddings, LayerNorm,
residuals).  The gather of the FP8 activations in front of a column-parallel GEMM and the
reduce-scatter behind a row-parallel GEMM run inside the GEMM kernels
(``msamp.parallel.fused.FusedGemmContext``), which is the B200 counterpart of the communication in the
reference's ``FP8LinearWithGradAccumulationAndAsyncCommunication`` (msamp/megatron/layers.py:52-219).

Tokens are kept in ``(batch, sequence)`` order and the flattened token axis is what is sharded: the
token-wise regions do not care which tokens a rank owns, and the gathered ``[tokens, features]``
matrix is in the order attention needs.

Parameters that are replicated over the group but see only this rank's tokens (LayerNorm weights,
embeddings, biases of the row-parallel layers) carry ``sequence_parallel = True``; their gradients are
partial sums and ``allreduce_sequence_parallel_grads`` adds them up over the group before the
optimizer (or the data-parallel reduction) runs, as Megatron does for such parameters.
"""
import math

import torch
import torch.distributed as dist
import torch.nn as nn

from msamp.megatron import parallel_state as mpu
from msamp.megatron.layers import ColumnParallelLinear, RowParallelLinear
from msamp.models.gpt import LayerNorm
from msamp.ops import nn as K


class _VocabParallelCrossEntropy(torch.autograd.Function):
    """Mean token cross-entropy of logits whose vocabulary axis is split over the tensor-parallel group."""
    @staticmethod
    def forward(ctx, logits, labels, vocab_start):
        group = mpu.get_tensor_model_parallel_group()
        tp = mpu.get_tensor_model_parallel_world_size()
        lf = logits.to(torch.float32, copy=True)
        m = lf.max(dim=-1).values
        if tp > 1:
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        lf.sub_(m.unsqueeze(-1))
        local = labels - vocab_start
        mine = (local >= 0) & (local < lf.shape[-1])
        picked = lf.gather(1, local.clamp(0, lf.shape[-1] - 1).unsqueeze(1)).squeeze(1)
        picked = torch.where(mine, picked, torch.zeros_like(picked))
        lf.exp_()
        denom = lf.sum(dim=-1)
        if tp > 1:
            dist.all_reduce(denom, group=group)
            dist.all_reduce(picked, group=group)
        loss = (denom.log() - picked).mean()
        lf.div_(denom.unsqueeze(-1))    # softmax over the full vocabulary, this rank's columns
        ctx.save_for_backward(lf, local, mine)
        ctx.in_dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, dloss):
        soft, local, mine = ctx.saved_tensors
        rows = soft.shape[0]
        grad = soft    # the saved buffer is not needed again
        idx = local.clamp(0, soft.shape[-1] - 1).unsqueeze(1)
        grad.scatter_add_(1, idx, -mine.to(grad.dtype).unsqueeze(1))
        grad.mul_(dloss / rows)
        return grad.to(ctx.in_dtype), None, None


def vocab_parallel_cross_entropy(logits, labels, vocab_start):
    return _VocabParallelCrossEntropy.apply(logits, labels, vocab_start)


class ParallelBlock(nn.Module):
    def __init__(self, cfg, device=None, sequence_parallel=True):
        super().__init__()
        tp = mpu.get_tensor_model_parallel_world_size()
        h, f = cfg.hidden, cfg.ffn_hidden
        if cfg.n_head % tp:
            raise ValueError(f'{cfg.n_head} heads cannot be split over {tp} tensor-parallel ranks')
        self.local_heads, self.head_dim = cfg.n_head // tp, cfg.head_dim
        sp = sequence_parallel
        proj_std = cfg.init_std / math.sqrt(2 * cfg.n_layer)
        self.ln1 = LayerNorm(h, cfg.eps, device)
        self.qkv = ColumnParallelLinear(h, 3 * h, sequence_parallel=sp, init_std=cfg.init_std, device=device)
        self.proj = RowParallelLinear(h, h, sequence_parallel=sp, init_std=proj_std, device=device)
        self.ln2 = LayerNorm(h, cfg.eps, device)
        self.fc1 = ColumnParallelLinear(h, f, sequence_parallel=sp, init_std=cfg.init_std, device=device)
        self.fc2 = RowParallelLinear(f, h, sequence_parallel=sp, init_std=proj_std, device=device)

    def forward(self, x, batch, seq):
        # x: [tokens / tp, hidden] (sequence parallel) or [tokens, hidden]
        qkv = self.qkv(self.ln1(x)).view(batch, seq, 3, self.local_heads, self.head_dim)
        o = K.attention_qkv(qkv, causal=True)
        x = x + self.proj(o.view(batch * seq, -1))
        x = x + self.fc2(K.gelu(self.fc1(self.ln2(x))))
        return x


class ParallelGPT(nn.Module):
    """Tensor- and sequence-parallel GPT.  ``forward(tokens, labels)`` returns the mean token loss.

    ``msamp.megatron.parallel_state.initialize_model_parallel`` must have been called; every rank of a
    tensor-parallel group must receive the same ``tokens`` and ``labels``.
    """
    def __init__(self, cfg, device=None, act_dtype=torch.bfloat16, sequence_parallel=True):
        super().__init__()
        self.cfg, self.act_dtype = cfg, act_dtype
        self.tp = mpu.get_tensor_model_parallel_world_size()
        self.tp_rank = mpu.get_tensor_model_parallel_rank()
        self.sequence_parallel = sequence_parallel and self.tp > 1
        if cfg.vocab_size % self.tp:
            raise ValueError('vocab_size must be divisible by the tensor-parallel size')
        self.wte = nn.Embedding(cfg.vocab_size, cfg.hidden, device=device, dtype=act_dtype)
        self.wpe = nn.Embedding(cfg.max_seq, cfg.hidden, device=device, dtype=act_dtype)
        self.blocks = nn.ModuleList(ParallelBlock(cfg, device, self.sequence_parallel) for _ in range(cfg.n_layer))
        self.ln_f = LayerNorm(cfg.hidden, cfg.eps, device)
        self.lm_head = ColumnParallelLinear(cfg.hidden, cfg.vocab_size, bias=False, sequence_parallel=self.sequence_parallel,
                                            init_std=cfg.init_std, device=device)
        with torch.no_grad():
            self.wte.weight.normal_(0.0, cfg.init_std)
            self.wpe.weight.normal_(0.0, cfg.init_std)
        if self.tp > 1:
            # identical replicas: start from rank 0's values
            for p in self.replicated_parameters():
                dist.broadcast(p.data, src=mpu.get_tensor_model_parallel_src_rank(), group=mpu.get_tensor_model_parallel_group())
        for p in self.replicated_parameters():
            p.sequence_parallel = self.sequence_parallel

    def replicated_parameters(self):
        """Parameters every rank of the tensor-parallel group holds in full."""
        out = [self.wte.weight, self.wpe.weight, self.ln_f.weight, self.ln_f.bias]
        for b in self.blocks:
            out += [b.ln1.weight, b.ln1.bias, b.ln2.weight, b.ln2.bias]
            out += [m.bias for m in (b.proj, b.fc2) if m.bias is not None]
        return out

    def allreduce_sequence_parallel_grads(self):
        """Sum the partial gradients of the replicated parameters over the tensor-parallel group."""
        if not self.sequence_parallel:
            return
        # Megatron-style local DDP accumulates into ``main_grad`` and leaves ``grad`` empty
        grads = [getattr(p, 'main_grad', None) if getattr(p, 'main_grad', None) is not None else p.grad
                 for p in self.replicated_parameters()]
        grads = [g for g in grads if g is not None]
        if not grads:
            return
        group = mpu.get_tensor_model_parallel_group()
        by_dtype = {}
        for g in grads:
            by_dtype.setdefault(g.dtype, []).append(g)
        for gs in by_dtype.values():
            flat = torch.cat([g.reshape(-1) for g in gs])
            dist.all_reduce(flat, group=group)
            off = 0
            for g in gs:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()

    def forward(self, tokens, labels=None):
        batch, seq = tokens.shape
        total = batch * seq
        flat = tokens.reshape(-1)
        pos = torch.arange(seq, device=tokens.device).repeat(batch)
        if self.sequence_parallel:
            if total % self.tp:
                raise ValueError('batch * seq must be divisible by the tensor-parallel size')
            n = total // self.tp
            sl = slice(self.tp_rank * n, (self.tp_rank + 1) * n)
            flat, pos = flat[sl], pos[sl]
        x = self.wte(flat) + self.wpe(pos)
        for blk in self.blocks:
            x = blk(x, batch, seq)
        logits = self.lm_head(self.ln_f(x))    # [tokens, vocab / tp]
        if labels is None:
            return logits
        v_local = self.cfg.vocab_size // self.tp
        return vocab_parallel_cross_entropy(logits, labels.reshape(-1), self.tp_rank * v_local)
