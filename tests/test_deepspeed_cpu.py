"""msamp.deepspeed on CPU: config parsing, engine selection, loss decrease with/without ZeRO, checkpoints, pipeline."""
import tempfile

import pytest
import torch
import torch.distributed as dist

from msamp import deepspeed
from msamp.deepspeed.runtime.config import MSAMPDeepSpeedConfig
from msamp.deepspeed.runtime.fp8.fused_optimizer import FP8Optimizer
from msamp.deepspeed.runtime.zero.fp8_stage_1_and_2 import FP8DeepSpeedZeroOptimizer
from msamp.optim import LBAdamW
from tests.dist_utils import run_workers


def _cfg(level='O2', zero=0, **extra):
    cfg = {
        'train_batch_size': 8, 'train_micro_batch_size_per_gpu': 4,
        'optimizer': {'type': 'AdamW', 'params': {'lr': 1e-2, 'weight_decay': 0.01}},
        'zero_optimization': {'stage': zero},
        'msamp': {'enabled': True, 'opt_level': level},
        'gradient_clipping': 1.0, 'wall_clock_breakdown': True, 'steps_per_print': 1000,
    }
    cfg.update(extra)
    return cfg


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 4))


def test_config_parsing_and_checks():
    c = MSAMPDeepSpeedConfig(_cfg())
    assert c.msamp_enabled and c.msamp_optlevel == 'O2' and c.gradient_accumulation_steps == 2 and not c.msamp_use_te
    assert not MSAMPDeepSpeedConfig({'train_batch_size': 4}).msamp_enabled
    with pytest.raises(AssertionError):
        MSAMPDeepSpeedConfig(_cfg(level='O3', zero=0))
    with pytest.raises(AssertionError):
        MSAMPDeepSpeedConfig(_cfg(level='O7'))
    with pytest.raises(AssertionError):
        MSAMPDeepSpeedConfig({'train_batch_size': 8, 'train_micro_batch_size_per_gpu': 3, 'gradient_accumulation_steps': 1})


@pytest.mark.parametrize('level,zero,cls', [('O1', 0, FP8Optimizer), ('O2', 0, FP8Optimizer), ('O2', 1, FP8DeepSpeedZeroOptimizer),
                                            ('O3', 2, FP8DeepSpeedZeroOptimizer)])
def test_engine_selection_and_training(level, zero, cls):
    engine, opt, _, _ = deepspeed.initialize(model=_model(), config=_cfg(level, zero))
    assert type(opt) is cls and isinstance(opt.optimizer, LBAdamW)
    x, y = torch.randn(32, 16), torch.randn(32, 4)
    losses = []
    for epoch in range(10):
        for i in range(0, 32, 4):
            loss = ((engine(x[i:i + 4]) - y[i:i + 4])**2).mean()
            engine.backward(loss)
            engine.step()
        losses.append(((engine(x) - y)**2).mean().item())
    assert losses[-1] < losses[0]
    assert engine.global_steps == 40 and engine.micro_steps == 80
    assert 'forward' in engine.timers.summary()
    with tempfile.TemporaryDirectory() as d:
        engine.save_checkpoint(d, tag='t')
        before = [p.float().clone() for p in engine.module.parameters()]
        engine.load_checkpoint(d)
        for a, b in zip(before, engine.module.parameters()):
            assert torch.allclose(a, b.float(), atol=1e-2)
    sd = opt.state_dict()
    assert {'dynamic_loss_scale', 'cur_scale', 'optimizer_state_dict', 'fp32_groups_flat', 'fp8_master_groups', 'clip_grad'} <= set(sd)
    if cls is FP8DeepSpeedZeroOptimizer:
        assert 'single_partition_of_fp8_groups' in sd


def test_dynamic_loss_scale_skips_overflow():
    cfg = _cfg('O2', 0, fp16={'enabled': True, 'loss_scale': 0, 'initial_scale_power': 4, 'hysteresis': 1})
    engine, opt, _, _ = deepspeed.initialize(model=_model(), config=cfg)
    assert opt.dynamic_loss_scale and opt.cur_scale == 16
    x = torch.randn(4, 16)
    w0 = engine.module[0].weight.float().clone()
    for _ in range(2):
        engine.backward(engine(x).mean() * float('inf'))    # every gradient becomes inf/nan
        engine.step()
    assert engine.skipped_steps == 1 and opt.cur_scale == 8
    assert torch.equal(w0, engine.module[0].weight.float())


def test_plain_engine_without_msamp():
    cfg = {'train_batch_size': 4, 'optimizer': {'type': 'Adam', 'params': {'lr': 1e-2}}}
    engine, opt, _, _ = deepspeed.initialize(model=_model(), config=cfg)
    assert isinstance(opt, torch.optim.Adam)
    loss = engine(torch.randn(4, 16)).square().mean()
    engine.backward(loss)
    engine.step()
    assert engine.global_steps == 1


def _pipeline(rank, world):
    from msamp.deepspeed import PipelineModule
    torch.manual_seed(0)
    layers = [torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 32), torch.nn.GELU(), torch.nn.Linear(32, 4)]
    pipe = PipelineModule(layers, num_stages=2, loss_fn=lambda out, y: ((out - y)**2).mean())
    cfg = {'train_batch_size': 8, 'train_micro_batch_size_per_gpu': 4, 'optimizer': {'type': 'AdamW', 'params': {'lr': 1e-2}},
           'msamp': {'enabled': True, 'opt_level': 'O2'}}
    engine, _, _, _ = deepspeed.initialize(model=pipe, config=cfg)
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(8, 16, generator=g), torch.randn(8, 4, generator=g)

    def batches():
        while True:
            yield x[:4], y[:4]
            yield x[4:], y[4:]

    it = batches()
    losses = [engine.train_batch(it).item() for _ in range(15)]
    if pipe.is_last_stage:
        assert losses[-1] < losses[0], losses
    assert len(list(pipe.layers)) in (2, 3)


def test_pipeline_engine_two_stages():
    run_workers(_pipeline, 2)


def _pipeline_1f1b(rank, world, enabled):
    """Four stages, six micro-batches: warm-up, steady and cool-down phases all occur; the result matches one process."""
    from msamp.deepspeed import PipelineModule
    torch.manual_seed(0)
    dims = [16, 32, 32, 32, 32, 32, 32, 32, 4]
    layers = []
    for i in range(8):
        layers.append(torch.nn.Sequential(torch.nn.Linear(dims[i], dims[i + 1]), torch.nn.Tanh()) if i < 7 else torch.nn.Linear(dims[i], dims[i + 1]))
    ref = torch.nn.Sequential(*[__import__('copy').deepcopy(l) for l in layers])
    loss_fn = lambda out, y: ((out - y)**2).mean()    # noqa: E731
    pipe = PipelineModule(layers, num_stages=4, loss_fn=loss_fn)
    cfg = {'train_batch_size': 24, 'train_micro_batch_size_per_gpu': 4, 'optimizer': {'type': 'AdamW', 'params': {'lr': 1e-2}},
           'gradient_clipping': 0.3, 'msamp': {'enabled': enabled, 'opt_level': 'O2'}}
    engine, _, _, _ = deepspeed.initialize(model=pipe, config=cfg)
    assert engine.gradient_accumulation_steps() == 6
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(24, 16, generator=g), torch.randn(24, 4, generator=g)

    def batches():
        while True:
            for i in range(6):
                yield x[4 * i:4 * i + 4], y[4 * i:4 * i + 4]

    it = batches()
    losses = [engine.train_batch(it).item() for _ in range(8)]
    if pipe.is_last_stage:
        assert losses[-1] < losses[0], losses
        if not enabled:
            opt = torch.optim.AdamW(ref.parameters(), lr=1e-2)
            want = []
            for _ in range(8):
                opt.zero_grad()
                total = 0.0
                for i in range(6):
                    lo = loss_fn(ref(x[4 * i:4 * i + 4]), y[4 * i:4 * i + 4]) / 6
                    lo.backward()
                    total += lo.item()
                torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.3)    # one norm over the whole model, as the stages must compute it
                opt.step()
                want.append(total)
            assert max(abs(a - b) for a, b in zip(losses, want)) < 1e-4, (losses, want)


def test_pipeline_1f1b_four_stages_fp8():
    run_workers(_pipeline_1f1b, 4, args=(True, ))


def test_pipeline_1f1b_matches_single_process():
    run_workers(_pipeline_1f1b, 4, args=(False, ))


def _engine_two_ranks(rank, world, level, zero, fp16):
    """The engine on two ranks: replicas stay identical under clipping (and dynamic loss scaling), loss falls."""
    extra = {'train_batch_size': 16}
    if fp16:
        extra['fp16'] = {'enabled': True, 'initial_scale_power': 8}
    engine, opt, _, _ = deepspeed.initialize(model=_model(), config=_cfg(level, zero, **extra))
    assert engine.gradient_accumulation_steps() == 2
    torch.manual_seed(3)
    x, y = torch.randn(64, 16), torch.randn(64, 4) * 3    # large targets: clipping at 1.0 is active
    lo = rank * 32
    first = last = None
    for epoch in range(6):
        for i in range(0, 32, 4):
            loss = ((engine(x[lo + i:lo + i + 4]) - y[lo + i:lo + i + 4])**2).mean()
            engine.backward(loss)
            engine.step()
        full = ((engine(x) - y)**2).mean().item()
        first = full if first is None else first
        last = full
    assert last < first
    flat = torch.cat([p.float().reshape(-1) for p in engine.module.parameters()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref), (flat - ref).abs().max()


@pytest.mark.parametrize('level,zero,fp16', [('O2', 0, False), ('O2', 1, False), ('O3', 2, False), ('O2', 2, True)])
def test_engine_two_ranks_replicas_agree(level, zero, fp16):
    run_workers(_engine_two_ranks, 2, args=(level, zero, fp16))


def _pipeline_with_dp(rank, world):
    """Two stages x two data-parallel replicas: replicas of a stage stay identical, loss falls."""
    from msamp.deepspeed import PipelineModule
    torch.manual_seed(0)
    layers = [torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 32), torch.nn.GELU(), torch.nn.Linear(32, 4)]
    pipe = PipelineModule(layers, num_stages=2, loss_fn=lambda out, y: ((out - y)**2).mean())
    assert pipe.dp_size == 2 and pipe.stage_id == rank // 2
    cfg = {'train_batch_size': 16, 'train_micro_batch_size_per_gpu': 4, 'optimizer': {'type': 'AdamW', 'params': {'lr': 1e-2}},
           'gradient_clipping': 1.0, 'msamp': {'enabled': True, 'opt_level': 'O2'}}
    engine, _, _, _ = deepspeed.initialize(model=pipe, config=cfg)
    assert engine.gradient_accumulation_steps() == 2
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(16, 16, generator=g), torch.randn(16, 4, generator=g) * 3
    dp_rank = rank % 2

    def batches():
        while True:
            for i in range(2):
                lo = dp_rank * 8 + 4 * i
                yield x[lo:lo + 4], y[lo:lo + 4]

    it = batches()
    losses = [engine.train_batch(it).item() for _ in range(10)]
    if pipe.is_last_stage:
        assert losses[-1] < losses[0], losses
    flat = torch.cat([p.float().reshape(-1) for p in engine.module.parameters()])
    ref = flat.clone()
    dist.broadcast(ref, src=dist.get_global_rank(pipe.get_data_parallel_group(), 0), group=pipe.get_data_parallel_group())
    assert torch.equal(flat, ref), (flat - ref).abs().max()


def test_pipeline_two_stages_two_replicas():
    run_workers(_pipeline_with_dp, 4)


def _resume_two_ranks(rank, world, path, zero):
    """Save after 3 steps, go on for 2; a fresh engine that loads the checkpoint and does the same 2 steps ends up equal."""
    from msamp.nn import model_state
    torch.manual_seed(3)
    x, y = torch.randn(64, 16), torch.randn(64, 4)
    lo = rank * 32

    def steps(engine, first, n):
        for s in range(first, first + n):
            for i in (0, 4):    # two micro-batches per step
                j = lo + (8 * s + i) % 32
                loss = ((engine(x[j:j + 4]) - y[j:j + 4])**2).mean()
                engine.backward(loss)
                engine.step()

    cfg = _cfg('O2', zero, train_batch_size=16)
    engine, _, _, _ = deepspeed.initialize(model=_model(), config=cfg)
    steps(engine, 0, 3)
    engine.save_checkpoint(path, tag='s3')
    steps(engine, 3, 2)
    want = torch.cat([p.float().reshape(-1) for p in engine.module.parameters()])
    model_state.clear()
    torch.manual_seed(99)
    fresh = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 4))    # other initial values
    engine2, _, _, _ = deepspeed.initialize(model=fresh, config=cfg)
    engine2.load_checkpoint(path)
    assert engine2.global_steps == 3
    steps(engine2, 3, 2)
    got = torch.cat([p.float().reshape(-1) for p in engine2.module.parameters()])
    assert (got - want).abs().max().item() <= 2e-2 * want.abs().max().item(), (got - want).abs().max()


@pytest.mark.parametrize('zero', [0, 2])
def test_engine_resume_two_ranks(tmp_path, zero):
    run_workers(_resume_two_ranks, 2, args=(str(tmp_path), zero))


def test_scheduler_dataloader_and_train_batch():
    data = torch.utils.data.TensorDataset(torch.randn(32, 16), torch.randn(32, 4))

    class WithLoss(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.net = _model()

        def forward(self, x, y):
            return ((self.net(x) - y)**2).mean()

    cfg = _cfg('O2', 0, scheduler={'type': 'WarmupLR', 'params': {'warmup_min_lr': 0.0, 'warmup_max_lr': 1e-2, 'warmup_num_steps': 4}})
    engine, opt, loader, sched = deepspeed.initialize(model=WithLoss(), config=cfg, training_data=data)
    assert loader is not None and loader.batch_size == 4 and sched is not None
    assert engine.get_lr()[0] == 0.0
    it = iter(loader)
    losses = [engine.train_batch(it) for _ in range(4)]    # two micro-batches each
    assert engine.global_steps == 4 and engine.micro_steps == 8
    assert abs(engine.get_lr()[0] - 1e-2) < 1e-12 and all(l == l for l in losses)
    sd = sched.state_dict()
    sched.load_state_dict(sd)
    assert sched.get_lr()[0] == engine.get_lr()[0]
    with pytest.raises(ValueError):
        deepspeed.initialize(model=WithLoss(), config=_cfg('O2', 0, scheduler={'type': 'OneCycle', 'params': {}}))
