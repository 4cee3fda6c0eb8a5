"""Multi-GPU tests (run only when at least two GPUs are visible): symmetric memory, fused FP8 reduce, sharded optimizer."""
import pytest
import torch
import torch.distributed as dist

import msamp
from msamp.common.dtype import Dtypes
from tests.dist_utils import run_workers

pytestmark = pytest.mark.gpu
E4M3 = Dtypes.kfloat8_e4m3


def _need(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f'needs {n} GPUs')


def _symm_and_barrier(rank, world):
    from msamp.ops import native
    from msamp.parallel.symm import FlagPad, SymmetricBuffer
    buf = SymmetricBuffer(1 << 20)
    mine = buf.view(torch.float32)
    mine.fill_(float(rank + 1))
    torch.cuda.synchronize()
    dist.barrier()
    flags = FlagPad()
    flags.barrier()
    torch.cuda.synchronize()
    assert native.device_status() == 0
    # a wait that nobody satisfies gives up after its limit and reports it; the context stays usable
    flags.epoch += 5
    flags.barrier(slot=4, limit_seconds=0.2, announce=False)
    torch.cuda.synchronize()
    assert native.device_status() & 2
    assert mine.sum().item() == (rank + 1) * mine.numel()
    dist.barrier()
    buf.close()


def test_symmetric_memory_and_bounded_barrier():
    _need(2)
    run_workers(_symm_and_barrier, 2, backend='nccl')


def _mk_model(dev):
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 512), torch.nn.GELU(),
                               torch.nn.Linear(512, 64)).to(dev)


def _fused_reduce_matches_math(rank, world):
    from msamp.ops import native
    from msamp.parallel.zero import ZeroShardedOptimizer
    dev = torch.device('cuda', rank)
    model = _mk_model(dev)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    model, opt = msamp.initialize(model, opt, 'O2')
    zero = ZeroShardedOptimizer(model, opt, stage=0)
    assert zero.native
    torch.manual_seed(100 + rank)
    x = torch.randn(64, 256, device=dev)
    model(x).square().mean().backward()
    # expected mean of the dequantised per-rank gradients
    expect = []
    for p in zero.fp8_params:
        g = p.grad.float()
        dist.all_reduce(g)
        expect.append(g / world)
    zero._reduce_fp8_grads()
    torch.cuda.synchronize()
    assert native.device_status() == 0
    for p, e in zip(zero.fp8_params, expect):
        got = p.grad.float()
        tol = 0.07 * e.abs().max().item() + 1e-8    # one e4m3 rounding of the mean
        assert (got - e).abs().max().item() <= tol
    # all ranks hold identical bytes and scales after the all-reduce flavour
    flat = zero.g_flat.clone()
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref)


def test_fused_fp8_allreduce():
    _need(2)
    run_workers(_fused_reduce_matches_math, 2, backend='nccl')


def _zero2_training(rank, world):
    from msamp.ops import native
    from msamp.parallel import DataParallelTrainer
    dev = torch.device('cuda', rank)
    model = _mk_model(dev)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    model, opt = msamp.initialize(model, opt, 'O2')

    class Wrap(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m

        def forward(self, x, y):
            return (self.m(x) - y).square().mean()

    wrapped = Wrap(model)
    trainer = DataParallelTrainer(wrapped, opt, zero_stage=2)
    torch.manual_seed(7)
    xs, ys = torch.randn(world * 32, 256, device=dev), torch.randn(world * 32, 64, device=dev)
    losses = []
    for _ in range(20):
        loss = trainer.step(xs[rank * 32:(rank + 1) * 32], ys[rank * 32:(rank + 1) * 32])
        losses.append(loss.item())
    torch.cuda.synchronize()
    assert native.device_status() == 0
    assert losses[-1] < 0.7 * losses[0], losses
    flat = torch.cat([p.float().reshape(-1) for p in model.parameters()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref)


def test_zero2_training_two_gpus():
    _need(2)
    run_workers(_zero2_training, 2, backend='nccl')
