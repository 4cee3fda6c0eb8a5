"""GPT pre-training on synthetic tokens with FP8 (O2) and optional ZeRO sharding over the node's GPUs.

    python examples/gpt_pretrain.py --model gpt-1.3b --steps 20
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 examples/gpt_pretrain.py --model gpt-7b --zero-stage 2
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..'))    # run from a source checkout without installing
import argparse

import torch
import torch.distributed as dist

import msamp
from msamp.models import GPT, gpt_config
from msamp.parallel import DataParallelTrainer
from msamp.utils import StepMetrics


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='gpt-small')
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--micro-batch', type=int, default=4)
    ap.add_argument('--seq', type=int, default=2048)
    ap.add_argument('--opt-level', default='O2')
    ap.add_argument('--zero-stage', type=int, default=2)
    ap.add_argument('--lr', type=float, default=3e-4)
    ap.add_argument('--clip', type=float, default=1.0)
    ap.add_argument('--metrics', default=None, help='JSONL file for per-step metrics')
    ap.add_argument('--recompute', action='store_true', help='re-run block forwards in backward instead of storing activations')
    ap.add_argument('--cpu', action='store_true', help='run the bit-exact CPU emulation (gloo for more than one rank)')
    args = ap.parse_args()
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    if args.cpu:
        dev = torch.device('cpu')
    else:
        torch.cuda.set_device(local)
        dev = torch.device('cuda', local)
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        if args.cpu:
            dist.init_process_group('gloo')
        else:
            dist.init_process_group('nccl', device_id=dev)
    rank = dist.get_rank() if world > 1 else 0
    cfg = gpt_config(args.model, max_seq=args.seq, recompute=args.recompute)
    model = GPT(cfg, device=dev, act_dtype=torch.float32 if args.cpu else torch.bfloat16)
    opt = torch.optim.AdamW(model.parameters(), lr=args.lr, betas=(0.9, 0.95), weight_decay=0.1)
    model, opt = msamp.initialize(model, opt, args.opt_level)
    trainer = DataParallelTrainer(model, opt, zero_stage=args.zero_stage if world > 1 else 0, clip_grad=args.clip)
    metrics = StepMetrics(args.metrics, rank)
    g = torch.Generator().manual_seed(rank)
    for step in range(args.steps):
        tok = torch.randint(0, cfg.vocab_size, (args.micro_batch, args.seq), generator=g)
        tok = tok if args.cpu else tok.pin_memory().to(dev, non_blocking=True)
        loss = trainer.step(tok, tok.roll(-1, 1))
        if step % 5 == 0:
            rec = metrics.log(step, tokens=args.micro_batch * args.seq * world * 5, loss=loss.item())
            if rank == 0:
                print(rec)
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
