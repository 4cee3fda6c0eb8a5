"""The MNIST-shaped CNN under FP8 DistributedDataParallel.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/mnist_ddp.py --opt-level O1
    (CPU: add --cpu to use the gloo backend and the FP8 emulation.)
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..'))    # run from a source checkout without installing
import argparse
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F

import msamp
from mnist import Net, synthetic_loader


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--opt-level', default='O1')
    ap.add_argument('--batches', type=int, default=30)
    ap.add_argument('--batch-size', type=int, default=64)
    ap.add_argument('--cpu', action='store_true')
    args = ap.parse_args()
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    use_cuda = torch.cuda.is_available() and not args.cpu
    if not use_cuda:
        os.environ['MSAMP_DEVICE'] = 'cpu'
    dist.init_process_group('nccl' if use_cuda else 'gloo')
    rank = dist.get_rank()
    device = torch.device('cuda', int(os.environ.get('LOCAL_RANK', 0))) if use_cuda else torch.device('cpu')
    if use_cuda:
        torch.cuda.set_device(device)
    model = Net().to(device)
    optimizer = torch.optim.Adam(model.parameters(), lr=1e-3)
    model, optimizer = msamp.initialize(model, optimizer, opt_level=args.opt_level)
    # importing msamp made torch.nn.parallel.DistributedDataParallel FP8-aware
    model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[device.index] if use_cuda else None)
    for i, (x, y) in enumerate(synthetic_loader(args.batches, args.batch_size, device, seed=rank)):
        optimizer.zero_grad()
        loss = F.nll_loss(model(x), y)
        loss.backward()
        optimizer.all_reduce_grads(model)    # no-op here: the FP8 DDP reducer already averaged the FP8 weight gradients
        optimizer.step()
        if rank == 0 and i % 10 == 0:
            print(f'batch {i} loss {loss.item():.4f}')
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
