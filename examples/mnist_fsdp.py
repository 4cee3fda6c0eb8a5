"""The MNIST-shaped CNN with its linears fully sharded (ZeRO-3 style) over the data-parallel group.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/mnist_fsdp.py
    torchrun ... examples/mnist_fsdp.py --torch-fsdp     # torch's own FSDP carrying the FP8 bytes, with FSDPAdamW
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..'))    # run from a source checkout without installing
import argparse

import torch
import torch.distributed as dist
import torch.nn.functional as F

from msamp.fsdp import FP8FullyShardedDataParallel
from mnist import Net, synthetic_loader


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--batches', type=int, default=30)
    ap.add_argument('--cpu', action='store_true')
    ap.add_argument('--torch-fsdp', action='store_true', help="use torch.distributed.fsdp with msamp's FP8 gradient hook")
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
    if args.torch_fsdp:
        from msamp.fsdp import wrap_with_torch_fsdp
        from msamp.optim import FSDPAdamW
        model = wrap_with_torch_fsdp(Net().to(device), device_id=device)
        optimizer = FSDPAdamW(model.parameters(), lr=1e-3)
    else:
        model = FP8FullyShardedDataParallel(Net().to(device))
        optimizer = model.build_optimizer(torch.optim.AdamW, lr=1e-3)
    for i, (x, y) in enumerate(synthetic_loader(args.batches, 64, device, seed=rank)):
        loss = F.nll_loss(model(x), y)
        loss.backward()
        if args.torch_fsdp:
            optimizer.step()
            optimizer.zero_grad(set_to_none=True)
        else:
            model.step(optimizer)
        if rank == 0 and i % 10 == 0:
            print(f'batch {i} loss {loss.item():.4f}')
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
