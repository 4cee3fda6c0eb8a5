"""Training-loss curves of a small GPT under fp32 and MS-AMP O1 / O2 / O3 on the same data and seeds.

    python benchmarks/loss_curves.py [--steps 300] [--device cpu|cuda] [--out curves.json]

The data are synthetic but learnable: each sequence follows a fixed random successor table with 10 % noise,
so the loss falls from ln(vocab) towards the entropy of the noise.  On the CPU the FP8 operators are the
bit-exact emulation of the CUDA kernels (the GEMM differs only in accumulation order).
"""
import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import msamp    # noqa: E402
from msamp.models import GPT, gpt_config    # noqa: E402


def batches(vocab, batch, seq, steps, seed):
    g = torch.Generator().manual_seed(seed)
    succ = torch.randperm(vocab, generator=g)
    for _ in range(steps):
        tok = torch.empty(batch, seq + 1, dtype=torch.long)
        tok[:, 0] = torch.randint(0, vocab, (batch, ), generator=g)
        for t in range(seq):
            nxt = succ[tok[:, t]]
            noise = torch.randint(0, vocab, (batch, ), generator=g)
            tok[:, t + 1] = torch.where(torch.rand(batch, generator=g) < 0.1, noise, nxt)
        yield tok[:, :-1], tok[:, 1:]


def run(level, args, dev):
    torch.manual_seed(0)
    cfg = gpt_config('gpt-tiny', n_layer=2, n_head=2, hidden=128, ffn_hidden=512, vocab_size=256, max_seq=args.seq)
    model = GPT(cfg, device=dev, act_dtype=torch.float32 if dev.type == 'cpu' else torch.bfloat16)
    opt = torch.optim.AdamW(model.parameters(), lr=args.lr, betas=(0.9, 0.95), weight_decay=0.01)
    if level != 'fp32':
        model, opt = msamp.initialize(model, opt, level)
    losses = []
    for x, y in batches(cfg.vocab_size, args.batch, args.seq, args.steps, seed=1):
        opt.zero_grad()
        loss = model(x.to(dev), y.to(dev))
        loss.backward()
        opt.step()
        losses.append(loss.detach().item())
    return losses


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--steps', type=int, default=300)
    ap.add_argument('--batch', type=int, default=8)
    ap.add_argument('--seq', type=int, default=64)
    ap.add_argument('--lr', type=float, default=3e-3)
    ap.add_argument('--device', default='cpu')
    ap.add_argument('--out', default=None)
    args = ap.parse_args()
    if args.device == 'cpu':
        os.environ['MSAMP_DEVICE'] = 'cpu'
    dev = torch.device(args.device)
    curves = {}
    for level in ('fp32', 'O1', 'O2', 'O3'):
        curves[level] = run(level, args, dev)
        c = curves[level]
        tail = sum(c[-20:]) / 20
        print(f'{level:5s} first {c[0]:.4f}  step {len(c) // 2}: {c[len(c) // 2]:.4f}  mean of last 20: {tail:.4f}', flush=True)
    ref = sum(curves['fp32'][-20:]) / 20
    for level in ('O1', 'O2', 'O3'):
        tail = sum(curves[level][-20:]) / 20
        print(f'{level}: final loss {tail:.4f} vs fp32 {ref:.4f} ({100 * (tail - ref) / ref:+.2f} %), ln(vocab) = {math.log(256):.3f}')
    if args.out:
        with open(args.out, 'w') as f:
            json.dump(curves, f)


if __name__ == '__main__':
    main()
