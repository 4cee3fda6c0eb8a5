"""GPT decoder (pre-LayerNorm, learned positions, GeLU MLP) on msamp's kernels.

Every projection is an ``nn.Linear`` so that ``msamp.initialize`` / ``LinearReplacer`` turns it into an
``FP8Linear``; LayerNorm, GeLU, causal attention and the loss use the kernels in ``msamp.ops.nn``.
The fused QKV projection output ``[tokens, 3*hidden]`` is read by the attention kernel through
strides and its gradient is produced in the same packed layout, so no split/concat copies exist.
"""
import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.utils.checkpoint

from msamp.nn import fused_layers as FL
from msamp.ops import nn as K


@dataclass
class GPTConfig:
    n_layer: int = 12
    n_head: int = 12
    hidden: int = 768
    ffn_hidden: int = 3072
    vocab_size: int = 50304
    max_seq: int = 2048
    eps: float = 1e-5
    init_std: float = 0.02
    tie_embeddings: bool = False
    recompute: bool = False    # re-run every block's forward during backward instead of keeping its activations

    @property
    def head_dim(self):
        return self.hidden // self.n_head

    def num_params(self):
        h, f, v = self.hidden, self.ffn_hidden, self.vocab_size
        per_layer = 4 * h * h + 2 * h * f + 4 * h + f + h + 4 * h
        return self.n_layer * per_layer + v * h * (1 if self.tie_embeddings else 2) + self.max_seq * h + 2 * h

    def flops_per_token(self, seq):
        """Model FLOPs per token for forward + backward (dense GEMMs x3, causal attention)."""
        h, f, v = self.hidden, self.ffn_hidden, self.vocab_size
        gemm = 2 * (4 * h * h + 2 * h * f) * self.n_layer + 2 * h * v
        attn = 2 * 2 * seq * h * self.n_layer / 2    # QK^T and PV, causal half
        return 3 * gemm + 3.5 * attn


_PRESETS = {
    'gpt-tiny': dict(n_layer=2, n_head=2, hidden=128, ffn_hidden=512, vocab_size=512, max_seq=128),
    'gpt-small': dict(n_layer=12, n_head=12, hidden=768, ffn_hidden=3072),
    'gpt-1.3b': dict(n_layer=24, n_head=16, hidden=2048, ffn_hidden=8192),
    'gpt-7b': dict(n_layer=32, n_head=32, hidden=4096, ffn_hidden=16384),
    'gpt-13b': dict(n_layer=40, n_head=40, hidden=5120, ffn_hidden=20480),
    'gpt-30b': dict(n_layer=48, n_head=56, hidden=7168, ffn_hidden=28672),
}


def gpt_config(name, **overrides):
    """Named configuration (``gpt-7b``, ``gpt-13b``, ``gpt-30b``, …) with optional field overrides."""
    cfg = dict(_PRESETS[name])
    cfg.update(overrides)
    return GPTConfig(**cfg)


class LayerNorm(nn.Module):
    """LayerNorm with fp32 affine parameters applied to activations of any floating dtype."""
    def __init__(self, hidden, eps=1e-5, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden, dtype=torch.float32, device=device))
        self.bias = nn.Parameter(torch.zeros(hidden, dtype=torch.float32, device=device))
        self.eps = eps

    def forward(self, x):
        return K.layer_norm(x, self.weight, self.bias, self.eps)


class Block(nn.Module):
    def __init__(self, cfg, device=None):
        super().__init__()
        h, f = cfg.hidden, cfg.ffn_hidden
        self.n_head, self.head_dim = cfg.n_head, cfg.head_dim
        self.ln1 = LayerNorm(h, cfg.eps, device)
        self.qkv = nn.Linear(h, 3 * h, device=device)
        self.proj = nn.Linear(h, h, device=device)
        self.ln2 = LayerNorm(h, cfg.eps, device)
        self.fc1 = nn.Linear(h, f, device=device)
        self.fc2 = nn.Linear(f, h, device=device)

    def forward(self, x, batch, seq):
        # x: [batch*seq, hidden]
        if FL.fusable(self.qkv, self.proj, self.fc1, self.fc2):
            # FP8 linears: each half of the block is one fused autograd function (msamp.nn.fused_layers)
            x = FL.attention_sublayer(x, self.ln1, self.qkv, self.proj, batch, seq, self.n_head, causal=True)
            return FL.mlp_sublayer(x, self.ln2, self.fc1, self.fc2)
        qkv = self.qkv(self.ln1(x)).view(batch, seq, 3, self.n_head, self.head_dim)
        o = K.attention_qkv(qkv, causal=True)
        x = x + self.proj(o.view(batch * seq, -1))
        x = x + self.fc2(K.gelu(self.fc1(self.ln2(x))))
        return x


class GPT(nn.Module):
    """Decoder-only language model. ``forward(tokens, labels)`` returns the mean token loss, else logits."""
    def __init__(self, cfg, device=None, act_dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        self.act_dtype = act_dtype
        self.wte = nn.Embedding(cfg.vocab_size, cfg.hidden, device=device, dtype=act_dtype)
        self.wpe = nn.Embedding(cfg.max_seq, cfg.hidden, device=device, dtype=act_dtype)
        self.blocks = nn.ModuleList(Block(cfg, device) for _ in range(cfg.n_layer))
        self.ln_f = LayerNorm(cfg.hidden, cfg.eps, device)
        self.lm_head = nn.Linear(cfg.hidden, cfg.vocab_size, bias=False, device=device)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self):
        std = self.cfg.init_std
        for name, p in self.named_parameters():
            if p.dim() < 2:
                if name.endswith('bias'):
                    p.zero_()
                continue
            if name.endswith('proj.weight') or name.endswith('fc2.weight'):
                p.normal_(0.0, std / math.sqrt(2 * self.cfg.n_layer))
            else:
                p.normal_(0.0, std)

    def forward(self, tokens, labels=None):
        batch, seq = tokens.shape
        pos = torch.arange(seq, device=tokens.device)
        x = (self.wte(tokens) + self.wpe(pos)).view(batch * seq, -1)
        for blk in self.blocks:
            if self.cfg.recompute and torch.is_grad_enabled():
                # the FP8 casts of the re-run see the same tensors and the same metas, so they repeat bit for bit
                x = torch.utils.checkpoint.checkpoint(blk, x, batch, seq, use_reentrant=False)
            else:
                x = blk(x, batch, seq)
        logits = FL.ln_linear(x, self.ln_f, self.lm_head) if FL.fusable(self.lm_head) else self.lm_head(self.ln_f(x))
        if labels is None:
            return logits.view(batch, seq, -1)
        return K.cross_entropy(logits, labels.reshape(-1))
