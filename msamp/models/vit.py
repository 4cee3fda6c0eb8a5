"""Vision Transformer classifier on msamp's kernels (the second model family next to GPT).

Patches are unfolded and projected by an ``nn.Linear`` (not a convolution), so that ``msamp.initialize``
turns every projection of the network, the patch embedding included, into an ``FP8Linear``.  Blocks are
pre-LayerNorm with bidirectional attention; LayerNorm, GeLU and attention use ``msamp.ops.nn``.
The reference publishes FP8 results for ViT / DeiT / Swin models trained with its O2 level
(docs/introduction.md:35-49); this module gives the same kind of workload a home in the framework.
"""
from dataclasses import dataclass

import torch
import torch.nn as nn

from msamp.models.gpt import LayerNorm
from msamp.ops import nn as K


@dataclass
class ViTConfig:
    image_size: int = 224
    patch_size: int = 16
    channels: int = 3
    n_layer: int = 12
    n_head: int = 12
    hidden: int = 768
    ffn_hidden: int = 3072
    num_classes: int = 1000
    eps: float = 1e-6
    init_std: float = 0.02

    @property
    def head_dim(self):
        return self.hidden // self.n_head

    @property
    def num_patches(self):
        return (self.image_size // self.patch_size)**2


_PRESETS = {
    'vit-tiny-test': dict(image_size=32, patch_size=8, n_layer=2, n_head=2, hidden=128, ffn_hidden=256, num_classes=10),
    'vit-s16': dict(n_layer=12, n_head=6, hidden=384, ffn_hidden=1536),
    'vit-b16': dict(n_layer=12, n_head=12, hidden=768, ffn_hidden=3072),
    'vit-l16': dict(n_layer=24, n_head=16, hidden=1024, ffn_hidden=4096),
    'vit-1.2b': dict(patch_size=14, n_layer=40, n_head=12, hidden=1536, ffn_hidden=6144),
}


def vit_config(name, **overrides):
    """Named configuration (``vit-b16``, ``vit-l16``, ``vit-1.2b``, …) with optional field overrides."""
    cfg = dict(_PRESETS[name])
    cfg.update(overrides)
    return ViTConfig(**cfg)


class ViTBlock(nn.Module):
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
        qkv = self.qkv(self.ln1(x)).view(batch, seq, 3, self.n_head, self.head_dim)
        o = K.attention_qkv(qkv, causal=False)
        x = x + self.proj(o.reshape(batch * seq, -1))
        x = x + self.fc2(K.gelu(self.fc1(self.ln2(x))))
        return x


class ViT(nn.Module):
    """``forward(images)`` returns logits ``[batch, classes]``; ``forward(images, labels)`` the mean loss."""
    def __init__(self, cfg, device=None, act_dtype=torch.bfloat16):
        super().__init__()
        self.cfg, self.act_dtype = cfg, act_dtype
        patch_dim = cfg.channels * cfg.patch_size * cfg.patch_size
        self.patch_embed = nn.Linear(patch_dim, cfg.hidden, device=device)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, cfg.hidden, device=device, dtype=act_dtype))
        self.pos_embed = nn.Parameter(torch.zeros(1, cfg.num_patches + 1, cfg.hidden, device=device, dtype=act_dtype))
        self.blocks = nn.ModuleList(ViTBlock(cfg, device) for _ in range(cfg.n_layer))
        self.ln_f = LayerNorm(cfg.hidden, cfg.eps, device)
        self.head = nn.Linear(cfg.hidden, cfg.num_classes, device=device)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self):
        for name, p in self.named_parameters():
            if name in ('cls_token', 'pos_embed') or (p.dim() >= 2 and name.endswith('weight')):
                p.normal_(0.0, self.cfg.init_std)
            elif name.endswith('bias'):
                p.zero_()

    def patches(self, images):
        """``[B, C, H, W]`` → ``[B, patches, C * p * p]`` (rows of one patch are contiguous)."""
        p = self.cfg.patch_size
        b, c, h, w = images.shape
        x = images.reshape(b, c, h // p, p, w // p, p).permute(0, 2, 4, 1, 3, 5)
        return x.reshape(b, (h // p) * (w // p), c * p * p)

    def forward(self, images, labels=None):
        x = self.patches(images.to(self.act_dtype))
        b, n, _ = x.shape
        x = self.patch_embed(x.reshape(b * n, -1)).view(b, n, -1)
        x = torch.cat([self.cls_token.expand(b, -1, -1).to(x.dtype), x], dim=1) + self.pos_embed.to(x.dtype)
        seq = n + 1
        x = x.reshape(b * seq, -1)
        for blk in self.blocks:
            x = blk(x, b, seq)
        x = self.ln_f(x).view(b, seq, -1)[:, 0]
        logits = self.head(x)
        if labels is None:
            return logits
        return torch.nn.functional.cross_entropy(logits.float(), labels)
