"""CIFAR10-shaped Vision Transformer on TE-style fused layers through the DeepSpeed-style engine.

The blocks are ``msamp.te.MSAMPTransformerLayer`` (LayerNorm→QKV, attention, proj, LayerNorm→MLP as fused FP8
modules with Transformer Engine's parameter names); with Transformer Engine installed the same script can build
``te.TransformerLayer`` blocks instead (``--use-te-modules``) and ``"use_te": true`` converts them.
Synthetic images unless --data-dir is given.  (reference: examples/cifar10_deepspeed_te.py)

    python examples/cifar10_deepspeed_te.py --deepspeed_config examples/ds_config_zero_te_msamp.json
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/cifar10_deepspeed_te.py
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..'))    # run from a source checkout without installing
import argparse

import torch
import torch.nn as nn
import torch.nn.functional as F

from msamp import deepspeed
from msamp.te import MSAMPTransformerLayer, te_available


class VisionTransformer(nn.Module):
    """Patch embedding, a stack of transformer layers, mean pooling and a classification head."""
    def __init__(self, image=32, patch=4, hidden=256, heads=4, ffn=1024, depth=4, classes=10, use_te_modules=False, dtype=torch.float32):
        super().__init__()
        self.patch, self.hidden, self.dtype = patch, hidden, dtype
        n_patches = (image // patch)**2
        self.embed = nn.Linear(3 * patch * patch, hidden)
        self.embed.use_fp32_linear = True    # the input projection stays in high precision
        self.pos = nn.Parameter(torch.zeros(n_patches, 1, hidden))
        if use_te_modules:
            import transformer_engine.pytorch as te
            make = lambda: te.TransformerLayer(hidden, ffn, heads, self_attn_mask_type='padding', hidden_dropout=0.0, attention_dropout=0.0)    # noqa: E731
        else:
            make = lambda: MSAMPTransformerLayer(hidden, ffn, heads, self_attn_mask_type='padding')    # noqa: E731
        self.layers = nn.ModuleList(make() for _ in range(depth))
        self.norm = nn.LayerNorm(hidden)
        self.head = nn.Linear(hidden, classes)
        self.head.use_fp32_linear = True
        nn.init.normal_(self.pos, std=0.02)

    def forward(self, x, y):
        b, p = x.shape[0], self.patch
        patches = x.unfold(2, p, p).unfold(3, p, p).permute(0, 2, 3, 1, 4, 5).reshape(b, -1, 3 * p * p)
        h = self.embed(patches).transpose(0, 1) + self.pos    # [patches, batch, hidden] as TE lays sequences out
        h = h.to(self.dtype)
        for layer in self.layers:
            h = layer(h)
        logits = self.head(self.norm(h.float().mean(0)))
        return F.cross_entropy(logits, y)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--deepspeed_config', default=os.path.join(os.path.dirname(__file__), 'ds_config_zero_te_msamp.json'))
    ap.add_argument('--steps', type=int, default=40)
    ap.add_argument('--depth', type=int, default=4)
    ap.add_argument('--hidden', type=int, default=256)
    ap.add_argument('--use-te-modules', action='store_true', help='build transformer_engine.pytorch.TransformerLayer blocks (needs TE)')
    ap.add_argument('--local_rank', type=int, default=int(os.environ.get('LOCAL_RANK', 0)))
    args = ap.parse_args()
    if args.use_te_modules and not te_available():
        raise SystemExit('--use-te-modules needs Transformer Engine; without it the script uses msamp.te.MSAMPTransformerLayer')
    distributed = int(os.environ.get('WORLD_SIZE', '1')) > 1
    device = torch.device('cuda', args.local_rank) if (torch.cuda.is_available() and os.environ.get('MSAMP_DEVICE') != 'cpu') else torch.device('cpu')
    if device.type == 'cuda':
        torch.cuda.set_device(device)
    dtype = torch.bfloat16 if device.type == 'cuda' else torch.float32
    heads = max(1, args.hidden // 64)
    model = VisionTransformer(hidden=args.hidden, heads=heads, ffn=4 * args.hidden, depth=args.depth, use_te_modules=args.use_te_modules,
                              dtype=dtype).to(device)
    engine, _, _, _ = deepspeed.initialize(args=args, model=model, dist_init_required=distributed)
    rank = getattr(engine, 'global_rank', 0)
    g = torch.Generator().manual_seed(rank)
    mb = engine.train_micro_batch_size_per_gpu()
    for step in range(args.steps * engine.gradient_accumulation_steps()):
        x = torch.randn(mb, 3, 32, 32, generator=g).to(device)
        y = torch.randint(0, 10, (mb, ), generator=g).to(device)
        loss = engine(x, y)
        engine.backward(loss)
        engine.step()
        if rank == 0 and step % 10 == 0:
            print(f'step {engine.global_steps} loss {loss.item():.4f} lr {engine.get_lr()[0]:.2e}')


if __name__ == '__main__':
    main()
