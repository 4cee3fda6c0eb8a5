"""The example scripts run end to end on the CPU emulation (a few steps each, synthetic data)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, nproc=1, timeout=420):
    env = dict(os.environ, MSAMP_DEVICE='cpu', MASTER_ADDR='127.0.0.1', OMP_NUM_THREADS='2')
    if nproc == 1:
        cmd = [sys.executable] + args
    else:
        cmd = [sys.executable, '-m', 'torch.distributed.run', '--standalone', '--local-addr', '127.0.0.1', '--nproc-per-node', str(nproc)] + args
    res = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return res.stdout


def test_mnist_single():
    out = _run(['examples/mnist.py', '--batches', '8', '--opt-level', 'O2'])
    assert 'loss' in out


@pytest.mark.parametrize('config', ['ds_config_msamp.json', 'ds_config_zero_te_msamp.json'])
def test_cifar10_deepspeed_config(config):
    out = _run(['examples/cifar10_deepspeed.py', '--steps', '4', '--deepspeed_config', os.path.join('examples', config)])
    assert 'loss' in out


def test_cifar10_deepspeed_te_vit():
    """Vision Transformer on msamp.te.MSAMPTransformerLayer with the ZeRO-2 + O3 + use_te configuration."""
    out = _run(['examples/cifar10_deepspeed_te.py', '--steps', '3', '--depth', '2', '--hidden', '128',
                '--deepspeed_config', os.path.join('examples', 'ds_config_zero_te_msamp.json')])
    assert 'loss' in out


def test_gpt_pretrain_tiny():
    out = _run(['examples/gpt_pretrain.py', '--cpu', '--model', 'gpt-tiny', '--steps', '6', '--seq', '64', '--micro-batch', '2'])
    assert "'loss'" in out


@pytest.mark.parametrize('script', ['examples/mnist_ddp.py', 'examples/mnist_fsdp.py'])
def test_mnist_two_ranks(script):
    out = _run([script, '--cpu', '--batches', '6'], nproc=2)
    assert 'loss' in out


def test_mnist_torch_fsdp_two_ranks():
    out = _run(['examples/mnist_fsdp.py', '--cpu', '--torch-fsdp', '--batches', '6'], nproc=2)
    assert 'loss' in out
