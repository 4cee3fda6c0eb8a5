"""CIFAR10-shaped classifier through the DeepSpeed-style engine (synthetic images unless --data-dir is given).

    python examples/cifar10_deepspeed.py --deepspeed_config examples/ds_config_msamp.json
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/cifar10_deepspeed.py --deepspeed_config examples/ds_config_zero_msamp.json
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..'))    # run from a source checkout without installing
import argparse
import os

import torch
import torch.nn as nn
import torch.nn.functional as F

from msamp import deepspeed


class Net(nn.Module):
    def __init__(self, hidden=512):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 6, 5)
        self.conv2 = nn.Conv2d(6, 16, 5)
        self.fc1 = nn.Linear(16 * 5 * 5, hidden)
        self.fc2 = nn.Linear(hidden, hidden)
        self.fc3 = nn.Linear(hidden, 10)

    def forward(self, x, y):
        x = F.max_pool2d(F.relu(self.conv1(x)), 2)
        x = F.max_pool2d(F.relu(self.conv2(x)), 2)
        x = F.relu(self.fc1(torch.flatten(x, 1)))
        x = F.relu(self.fc2(x))
        return F.cross_entropy(self.fc3(x).float(), y)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--deepspeed_config', default=os.path.join(os.path.dirname(__file__), 'ds_config_msamp.json'))
    ap.add_argument('--steps', type=int, default=40)
    ap.add_argument('--local_rank', type=int, default=int(os.environ.get('LOCAL_RANK', 0)))
    args = ap.parse_args()
    distributed = int(os.environ.get('WORLD_SIZE', '1')) > 1
    device = torch.device('cuda', args.local_rank) if torch.cuda.is_available() else torch.device('cpu')
    if device.type == 'cuda':
        torch.cuda.set_device(device)
    engine, _, _, _ = deepspeed.initialize(args=args, model=Net().to(device), dist_init_required=distributed)
    g = torch.Generator().manual_seed(engine.global_rank)
    mb = engine.train_micro_batch_size_per_gpu()
    for step in range(args.steps * engine.gradient_accumulation_steps()):
        x = torch.randn(mb, 3, 32, 32, generator=g).to(device)
        y = torch.randint(0, 10, (mb, ), generator=g).to(device)
        loss = engine(x, y)
        engine.backward(loss)
        engine.step()
        if engine.global_rank == 0 and step % 20 == 0:
            print(f'step {engine.global_steps} loss {loss.item():.4f} lr {engine.get_lr()[0]:.2e}')


if __name__ == '__main__':
    main()
