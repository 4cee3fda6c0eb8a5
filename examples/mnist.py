"""MNIST-shaped CNN trained with msamp (single process). Synthetic data by default; pass --data-dir for torchvision MNIST.

    python examples/mnist.py --opt-level O2 --epochs 1
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..'))    # run from a source checkout without installing
import argparse

import torch
import torch.nn as nn
import torch.nn.functional as F

import msamp


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 32, 3, 1)
        self.conv2 = nn.Conv2d(32, 64, 3, 1)
        self.fc1 = nn.Linear(9216, 128)
        self.fc2 = nn.Linear(128, 10)

    def forward(self, x):
        x = F.relu(self.conv1(x))
        x = F.max_pool2d(F.relu(self.conv2(x)), 2)
        x = F.relu(self.fc1(torch.flatten(x, 1)))
        return F.log_softmax(self.fc2(x), dim=1)


def synthetic_loader(n_batches, batch_size, device, seed=0):
    g = torch.Generator().manual_seed(seed)
    for _ in range(n_batches):
        yield torch.randn(batch_size, 1, 28, 28, generator=g).to(device), torch.randint(0, 10, (batch_size, ), generator=g).to(device)


def real_loader(data_dir, batch_size, device):
    from torchvision import datasets, transforms
    ds = datasets.MNIST(data_dir, train=True, download=False,
                        transform=transforms.Compose([transforms.ToTensor(), transforms.Normalize((0.1307, ), (0.3081, ))]))
    for x, y in torch.utils.data.DataLoader(ds, batch_size=batch_size, shuffle=True):
        yield x.to(device), y.to(device)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--opt-level', default='O1', choices=msamp.opt_levels)
    ap.add_argument('--epochs', type=int, default=1)
    ap.add_argument('--batch-size', type=int, default=64)
    ap.add_argument('--batches', type=int, default=50)
    ap.add_argument('--lr', type=float, default=1e-3)
    ap.add_argument('--data-dir', default=None)
    ap.add_argument('--no-msamp', action='store_true')
    args = ap.parse_args()
    device = torch.device('cuda' if torch.cuda.is_available() else 'cpu')
    model = Net().to(device)
    optimizer = torch.optim.AdamW(model.parameters(), lr=args.lr)
    if not args.no_msamp:
        model, optimizer = msamp.initialize(model, optimizer, opt_level=args.opt_level)
    scaler = torch.amp.GradScaler(device.type, enabled=device.type == 'cuda')
    for epoch in range(args.epochs):
        loader = real_loader(args.data_dir, args.batch_size, device) if args.data_dir else synthetic_loader(args.batches, args.batch_size, device, epoch)
        for i, (x, y) in enumerate(loader):
            optimizer.zero_grad()
            with torch.autocast(device.type, dtype=torch.bfloat16, enabled=device.type == 'cuda'):
                loss = F.nll_loss(model(x).float(), y)
            scaler.scale(loss).backward()
            scaler.step(optimizer)
            scaler.update()
            if i % 10 == 0:
                print(f'epoch {epoch} batch {i} loss {loss.item():.4f}')


if __name__ == '__main__':
    main()
