"""Times causal self-attention forward and backward on a packed ``[B, S, 3, heads, 128]`` tensor.

    python benchmarks/bench_attention.py [--batch 4] [--heads 32] [--seq 2048] [--iters 20] [--impl tc|mma|both]

Prints one line per implementation: milliseconds per call (launches queued back to back) and TFLOP/s (causal FLOPs: 4*B*H*S^2*d/2 forward,
2.5x that backward).  CUDA events, three warm-up iterations, L2 is not flushed (the working set of the
default case is 400 MB).
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from msamp.ops import native    # noqa: E402
from msamp.ops import nn as K    # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--batch', type=int, default=4)
    ap.add_argument('--heads', type=int, default=32)
    ap.add_argument('--seq', type=int, default=2048)
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='both')
    args = ap.parse_args()
    B, S, H, d = args.batch, args.seq, args.heads, 128
    qkv = torch.randn(B, S, 3, H, d, device='cuda').bfloat16().requires_grad_(True)
    do = torch.randn(B, S, H, d, device='cuda').bfloat16()
    flops = 4 * B * H * S * S * d / 2
    for impl in (['tc', 'mma'] if args.impl == 'both' else [args.impl]):
        os.environ['MSAMP_ATTN_IMPL'] = impl
        for _ in range(args.warmup):
            K.attention_qkv(qkv).backward(do)
        # launches are queued back to back (no host synchronisation inside a timed region)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        torch.cuda.synchronize()
        ev[0].record()
        with torch.no_grad():
            for _ in range(args.iters):
                K.attention_qkv(qkv)
        ev[1].record()
        torch.cuda.synchronize()
        outs = [K.attention_qkv(qkv) for _ in range(args.iters)]
        torch.cuda.synchronize()
        ev[2].record()
        for o in outs:
            torch.autograd.grad(o, qkv, do)
        ev[3].record()
        torch.cuda.synchronize()
        tf = ev[0].elapsed_time(ev[1]) / max(args.iters, 1)
        tb = ev[2].elapsed_time(ev[3]) / max(args.iters, 1)
        print(f'{impl}: B={B} H={H} S={S} fwd {tf:.3f} ms {flops / tf / 1e9:.0f} TFLOP/s | bwd {tb:.3f} ms '
              f'{2.5 * flops / tb / 1e9:.0f} TFLOP/s | device_status {native.device_status()}', flush=True)


if __name__ == '__main__':
    main()
