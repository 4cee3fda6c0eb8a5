"""Timers, step metrics and host-side failure detection (no GPU, no GPU fault: failures are made on the host)."""
import json
import time

import pytest
import torch
import torch.distributed as dist

from msamp.utils.heartbeat import Heartbeat, RankFailure
from msamp.utils.metrics import StepMetrics
from msamp.utils.timer import PhaseTimers, nvtx_range
from tests.dist_utils import run_workers


def test_phase_timers_accumulate_and_reset():
    timers = PhaseTimers()
    for _ in range(3):
        with timers.phase('basic_step'):
            time.sleep(0.002)
    timers('compute_norm').start()
    timers('compute_norm').stop()
    s = timers.summary()
    assert s['basic_step'] >= 1.5 and 'compute_norm' in s
    text = timers.log(names=['basic_step'])
    assert text.startswith('basic_step:') and 'compute_norm' not in text
    assert timers.summary()['basic_step'] == 0.0    # log() resets
    off = PhaseTimers(enabled=False)
    with off.phase('x'):
        pass
    assert off.summary() == {}
    with nvtx_range('noop'):
        pass


def test_step_metrics_jsonl(tmp_path):
    path = tmp_path / 'm.jsonl'
    m = StepMetrics(str(path), rank=3)
    time.sleep(0.001)
    m.skipped_steps = 2
    rec = m.log(7, tokens=4096, loss=torch.tensor(2.5), phases={'basic_step': 1.0}, lr=1e-4)
    assert rec['tokens_per_s'] > 0 and rec['loss'] == 2.5 and rec['skipped_steps'] == 2 and rec['lr'] == 1e-4
    line = json.loads(path.read_text().strip())
    assert line['step'] == 7 and line['rank'] == 3 and line['phases_ms'] == {'basic_step': 1.0}


def test_heartbeat_detects_a_silent_peer():
    store = dist.HashStore()
    a = Heartbeat(store, 0, 2, interval=0.02, timeout=0.15).start()
    b = Heartbeat(store, 1, 2, interval=0.02, timeout=0.15).start()
    try:
        time.sleep(0.1)
        a.check()
        b.check()
        b.stop()    # rank 1 "dies": its key stops changing
        deadline = time.time() + 3.0
        while time.time() < deadline and not a.stale_ranks():
            time.sleep(0.02)
        assert a.stale_ranks() == [1]
        with pytest.raises(RankFailure, match=r'ranks \[1\]'):
            a.check()
    finally:
        a.stop()
        b.stop()


def test_heartbeat_reports_peer_that_never_joined_and_device_status():
    store = dist.HashStore()
    hb = Heartbeat(store, 0, 3, interval=0.02, timeout=0.1)
    hb.check()    # inside the grace period nobody is stale
    time.sleep(0.25)
    assert hb.stale_ranks() == [1, 2]
    alone = Heartbeat(store, 0, 1)
    alone.check(device_status=0)
    with pytest.raises(RankFailure, match='device-side wait'):
        alone.check(device_status=2)


def _leaving_rank(rank, world):
    """Rank 1 leaves between steps; rank 0 learns of it from the store before its next collective."""
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval=0.05, timeout=0.4).start()
    x = torch.ones(4)
    for step in range(3):
        hb.check()
        dist.all_reduce(x)    # both ranks take part in three steps
    if rank == 1:
        hb.stop()    # stops beating and takes part in no further collective
        time.sleep(1.5)
    else:
        t0 = time.time()
        failed = False
        while time.time() - t0 < 5.0:
            try:
                hb.check()
            except RankFailure:
                failed = True
                break
            time.sleep(0.05)
        hb.stop()
        assert failed, 'rank 0 never noticed that rank 1 stopped'
        assert time.time() - t0 < 3.0


def test_rank_leaving_between_steps_is_seen_on_the_host():
    run_workers(_leaving_rank, world=2, backend='gloo')


def _trainer_stops_before_collective(rank, world):
    """Rank 1 stops after three steps; rank 0's trainer raises RankFailure instead of entering the next all-reduce."""
    import msamp
    from msamp.parallel import DataParallelTrainer
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval=0.05, timeout=0.4).start()
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 16), torch.nn.GELU(), torch.nn.Linear(16, 16))
    model, opt = msamp.initialize(model, torch.optim.AdamW(model.parameters(), lr=1e-3), 'O2')

    class _Loss(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m

        def forward(self, x, y):
            return ((self.m(x) - y)**2).mean()

    trainer = DataParallelTrainer(_Loss(model), opt, heartbeat=hb)
    x, y = torch.randn(8, 16), torch.randn(8, 16)
    for _ in range(3):
        trainer.step(x, y)
    if rank == 1:
        hb.stop()
        time.sleep(2.5)
        return
    deadline = time.time() + 5.0    # staleness counts from the last change this rank observed
    while time.time() < deadline and not hb.stale_ranks():
        time.sleep(0.05)
    assert hb.stale_ranks() == [1]
    with pytest.raises(RankFailure):
        trainer.step(x, y)
    hb.stop()


def test_trainer_checks_heartbeat_before_each_step():
    run_workers(_trainer_stops_before_collective, world=2, backend='gloo')
