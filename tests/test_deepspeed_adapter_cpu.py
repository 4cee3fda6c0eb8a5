"""msamp.deepspeed with a ``deepspeed`` package present: ``initialize`` must return a subclass of that package's engine.

DeepSpeed itself is not installed where these tests run; ``tests/fake_deepspeed`` provides a package with the engine /
config hooks the adapter relies on (see its docstring).  What is checked is the wiring: class hierarchy, optimizer
choice from the JSON config, the ``msamp`` section, gradient exchange left to the FP8 optimizers, and that a
facility of the host engine msamp's stand-alone engine lacks (here a scheduler type) keeps working.
"""
import os
import sys

import pytest
import torch

FAKE = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'fake_deepspeed')


@pytest.fixture
def fake_deepspeed():
    sys.path.insert(0, FAKE)
    for name in [m for m in sys.modules if m == 'deepspeed' or m.startswith('deepspeed.')]:
        del sys.modules[name]
    yield
    sys.path.remove(FAKE)
    for name in [m for m in sys.modules if m == 'deepspeed' or m.startswith('deepspeed.')]:
        del sys.modules[name]


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 4))


def _config(level='O2', stage=2, **extra):
    cfg = {'train_micro_batch_size_per_gpu': 8, 'gradient_accumulation_steps': 2, 'gradient_clipping': 1.0,
           'optimizer': {'type': 'AdamW', 'params': {'lr': 1e-2}},
           'scheduler': {'type': 'WarmupDecayLR', 'params': {'total_num_steps': 100, 'warmup_num_steps': 2, 'warmup_max_lr': 1e-2}},
           'zero_optimization': {'stage': stage}, 'msamp': {'enabled': True, 'opt_level': level}}
    cfg.update(extra)
    return cfg


def test_adapter_engine_subclasses_the_installed_engine(fake_deepspeed):
    from deepspeed.runtime.engine import DeepSpeedEngine
    from msamp import deepspeed as msamp_ds
    from msamp.deepspeed.runtime.adapter import deepspeed_available
    from msamp.deepspeed.runtime.fp8.fused_optimizer import FP8Optimizer
    from msamp.deepspeed.runtime.zero.fp8_stage_1_and_2 import FP8DeepSpeedZeroOptimizer
    from msamp.nn import FP8Linear
    assert deepspeed_available()
    engine, opt, _, sched = msamp_ds.initialize(model=_model(), config=_config('O2', 2))
    assert isinstance(engine, DeepSpeedEngine) and isinstance(opt, FP8DeepSpeedZeroOptimizer)
    assert isinstance(engine.module[0], FP8Linear) and engine._config.msamp_optlevel == 'O2'
    assert sched is not None and sched.get_lr()[0] == 0.0    # the host engine's own scheduler type
    x, y = torch.randn(64, 16), torch.randn(64, 4)
    losses = []
    for it in range(12):
        for micro in range(2):
            xb, yb = x[micro * 8:(micro + 1) * 8], y[micro * 8:(micro + 1) * 8]
            loss = ((engine(xb) - yb)**2).mean()
            engine.backward(loss)    # would raise in the host's allreduce_gradients if the adapter did not take it over
            engine.step()
        losses.append(loss.item())
    assert engine.global_steps == 12 and losses[-1] < losses[0]
    assert sched.get_lr()[0] > 0.0
    # no ZeRO -> FP8Optimizer; msamp disabled -> the host engine's own optimizer path
    engine2, opt2, _, _ = msamp_ds.initialize(model=_model(), config=_config('O1', 0))
    assert isinstance(opt2, FP8Optimizer) and not isinstance(opt2, FP8DeepSpeedZeroOptimizer)
    cfg = _config('O1', 0)
    cfg['msamp']['enabled'] = False
    engine3, opt3, _, _ = msamp_ds.initialize(model=_model(), config=cfg)
    assert isinstance(opt3, torch.optim.AdamW) and isinstance(engine3.module[0], torch.nn.Linear)


def test_adapter_config_checks(fake_deepspeed):
    from msamp import deepspeed as msamp_ds
    with pytest.raises(AssertionError, match='O3 requires ZeRO'):
        msamp_ds.initialize(model=_model(), config=_config('O3', 0))
    with pytest.raises(AssertionError, match='Invalid MS-AMP opt_level'):
        msamp_ds.initialize(model=_model(), config=_config('O9', 1))
    engine, opt, _, _ = msamp_ds.initialize(model=_model(), config=_config('O3', 1))
    assert opt.zero is not None and opt.zero.sharded


def test_without_deepspeed_the_standalone_engine_is_used():
    from msamp import deepspeed as msamp_ds
    from msamp.deepspeed.runtime.adapter import deepspeed_available
    if deepspeed_available():
        pytest.skip('a real DeepSpeed is installed')
    cfg = _config('O2', 2)
    cfg['scheduler'] = {'type': 'WarmupLR', 'params': {'warmup_num_steps': 2}}
    engine, _, _, _ = msamp_ds.initialize(model=_model(), config=cfg)
    assert isinstance(engine, msamp_ds.MSAMPDeepSpeedEngine)
