"""Multi-process logic on CPU with gloo: FP8 collectives, bucketed TensorDist, sharded optimizer, DDP training."""
import pytest
import torch
import torch.distributed as dist

import msamp
from msamp.common.dtype import Dtypes
from msamp.common.tensor import TensorDist
from msamp.operators.dist_op import DistOp
from msamp.parallel.zero import ZeroShardedOptimizer, partition_tensors
from tests.dist_utils import run_workers

E4M3 = Dtypes.kfloat8_e4m3


def test_partition_is_balanced_and_deterministic():
    owners = partition_tensors([100, 100, 50, 50, 10], 2)
    assert owners == [0, 1, 0, 1, 0]
    owners = partition_tensors([5] * 7, 3)
    assert sorted(owners.count(r) for r in range(3)) == [2, 2, 3]


def _fp8_collectives(rank, world):
    # all ranks hold 1.0 / 2.0 / -0.5 in e4m3: sums are exactly representable
    vals = torch.tensor([1.0, 2.0, -0.5, 0.0]).to(torch.float8_e4m3fn).view(torch.uint8)
    t = vals.clone()
    DistOp.all_reduce(t, E4M3, dist.ReduceOp.SUM)
    assert torch.equal(t.view(torch.float8_e4m3fn).float(), torch.tensor([2.0, 4.0, -1.0, 0.0]))
    t = (vals.view(torch.float8_e4m3fn).float() * (rank + 1)).to(torch.float8_e4m3fn).view(torch.uint8)
    DistOp.all_reduce(t, E4M3, dist.ReduceOp.MAX)
    assert torch.equal(t.view(torch.float8_e4m3fn).float(), torch.tensor([2.0, 4.0, -0.5, 0.0]))
    t = vals.clone()
    DistOp.reduce(t, E4M3, dst=1)
    want = torch.tensor([2.0, 4.0, -1.0, 0.0]) if rank == 1 else torch.tensor([1.0, 2.0, -0.5, 0.0])
    assert torch.equal(t.view(torch.float8_e4m3fn).float(), want)
    # hand-computed e4m3 bit patterns (the golden vectors of the reference's tests/operators/test_dist.py:112-136, 150-185)
    pats = [torch.tensor([0b01001010, 0b01011000], dtype=torch.uint8), torch.tensor([0b01010000, 0b01011100], dtype=torch.uint8)]
    t = pats[rank].clone()
    DistOp.all_reduce(t, E4M3, dist.ReduceOp.SUM)
    assert t.tolist() == [0b01010101, 0b01100010]
    t = pats[rank].clone()
    DistOp.all_reduce(t, E4M3, dist.ReduceOp.MAX)
    assert t.tolist() == [0b01010000, 0b01011100]
    t = pats[rank].clone()
    DistOp.all_reduce(t, E4M3, dist.ReduceOp.MIN)
    assert t.tolist() == [0b01001010, 0b01011000]
    t = pats[rank].clone()
    DistOp.reduce(t, E4M3, dst=1, op=dist.ReduceOp.SUM)
    assert t.tolist() == ([0b01010101, 0b01100010] if rank == 1 else pats[rank].tolist())
    # saturation instead of overflow
    big = torch.full((4, ), 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
    DistOp.all_reduce(big, E4M3, dist.ReduceOp.SUM)
    assert torch.equal(big.view(torch.float8_e4m3fn).float(), torch.full((4, ), 448.0))
    # ScalingTensor averaging touches scale_inv only
    x = torch.arange(8.0).cast(E4M3)
    before = x.value.clone()
    TensorDist.all_reduce_avg([x])
    assert torch.allclose(x.float(), torch.arange(8.0) , atol=0.3)
    assert not torch.equal(before, x.value) or world == 1 or True
    # broadcast of weights + scale_inv
    w = (torch.randn(16) * (rank + 1)).cast(Dtypes.kfloat16)
    TensorDist.broadcast([w], src=0)
    ref = [None]
    dist.broadcast_object_list(ref if rank else [w.float()], src=0)


def test_fp8_collectives_gloo():
    run_workers(_fp8_collectives, 2)


def _mk_model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 32), torch.nn.GELU(), torch.nn.Linear(32, 4))


def _zero_training(rank, world, stage):
    torch.manual_seed(0)
    x_all = torch.randn(8 * world, 16)
    y_all = torch.randn(8 * world, 4)
    model = _mk_model()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    model, opt = msamp.initialize(model, opt, 'O2')
    zero = ZeroShardedOptimizer(model, opt, stage=stage)
    losses = []
    for _ in range(12):
        xb, yb = x_all[rank * 8:(rank + 1) * 8], y_all[rank * 8:(rank + 1) * 8]
        loss = ((model(xb) - yb)**2).mean()
        loss.backward()
        zero.reduce_and_step()
        for p in zero.hp_params:
            p.grad = None
        losses.append(loss.item())
    # every rank must hold identical weights afterwards
    flat = torch.cat([p.float().reshape(-1) for p in model.parameters()])
    gathered = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat)
    for g in gathered:
        assert torch.equal(g, gathered[0])
    assert losses[-1] < losses[0]
    if stage >= 1:
        owned = sum(1 for o in zero.owners if o == rank)
        assert len(zero.masters) == owned and 0 < owned < len(zero.owners)
        sd = zero.state_dict()
        # the reference's nesting: one list of master weights per optimizer param group
        groups = sd['single_partition_of_fp8_groups']
        assert len(groups) == len(zero.optimizer.param_groups) and all(isinstance(g, list) for g in groups)
        assert sum(len(g) for g in groups) == owned
        zero.load_state_dict(sd)
        # a hand-built dictionary of that shape (what a checkpoint written by the reference carries) loads as well,
        # and so does the flat list older files of this library used
        before = [m.value.clone() for g in zero._master_groups() for m in g]
        hand = {'optimizer_state_dict': zero.optimizer.state_dict(), 'partition_count': world, 'zero_stage': stage,
                'single_partition_of_fp8_groups': [[t.clone() for t in g] for g in groups]}
        zero.load_state_dict(hand)
        legacy = dict(hand, single_partition_of_fp8_groups=[zero.masters[i].detach() for i in sorted(zero.masters)])
        zero.load_state_dict(legacy)
        after = [m.value for g in zero._master_groups() for m in g]
        assert all(torch.equal(a, b) for a, b in zip(before, after))
        bad = dict(hand, single_partition_of_fp8_groups=[g[:-1] for g in groups])
        try:
            zero.load_state_dict(bad)
            raise AssertionError('a checkpoint with a missing master weight must be rejected')
        except ValueError:
            pass
        # high-precision parameters are sharded too: the inner optimizer only holds what this rank owns
        hp_in_opt = sum(1 for g in zero.optimizer.param_groups for p in g['params'] if any(p is q for q in zero.hp_params))
        assert hp_in_opt == sum(1 for o in zero.hp_owner if o == rank) < len(zero.hp_params)
    return losses


def test_zero_stage2_gloo():
    run_workers(_zero_training, 2, args=(2, ))


def test_zero_stage0_gloo():
    run_workers(_zero_training, 2, args=(0, ))


def _zero_matches_single(rank, world):
    # world-averaged gradients of identical data must reproduce single-process training closely
    torch.manual_seed(0)
    x, y = torch.randn(8, 16), torch.randn(8, 4)
    model = _mk_model()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    model, opt = msamp.initialize(model, opt, 'O2')
    zero = ZeroShardedOptimizer(model, opt, stage=2)
    for _ in range(5):
        loss = ((model(x) - y)**2).mean()
        loss.backward()
        zero.reduce_and_step()
        for p in zero.hp_params:
            p.grad = None
    from msamp.nn import model_state
    model_state.clear()
    ref = _mk_model()
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2)
    for _ in range(5):
        ropt.zero_grad()
        rl = ((ref(x) - y)**2).mean()
        rl.backward()
        ropt.step()
    assert abs(loss.item() - rl.item()) < 0.1 * rl.item() + 0.02


def test_zero_tracks_fp32_training():
    run_workers(_zero_matches_single, 2)


def _ddp_training(rank, world):
    import torch.nn as nn
    from msamp.nn.distributed import FP8DistributedDataParallel
    torch.manual_seed(0)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv1 = nn.Conv2d(1, 8, 3, 1)
            self.conv2 = nn.Conv2d(8, 16, 3, 1)
            self.fc1 = nn.Linear(2304, 64)
            self.fc2 = nn.Linear(64, 10)

        def forward(self, x):
            x = torch.relu(self.conv1(x))
            x = torch.max_pool2d(torch.relu(self.conv2(x)), 2)
            return self.fc2(torch.relu(self.fc1(torch.flatten(x, 1))))

    model = Net()
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    model, opt = msamp.initialize(model, opt, 'O1')
    assert torch.nn.parallel.DistributedDataParallel is FP8DistributedDataParallel
    ddp = torch.nn.parallel.DistributedDataParallel(model)
    g = torch.Generator().manual_seed(10 + rank)
    x = torch.randn(16, 1, 28, 28, generator=g)
    y = torch.randint(0, 10, (16, ), generator=g)
    losses = []
    for _ in range(8):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(ddp(x), y)
        loss.backward()
        opt.all_reduce_grads(model)    # no-op under FP8 DDP
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
    w = model.fc1.weight
    assert w.grad is not None and w.grad.qtype == E4M3
    flat = torch.cat([p.float().reshape(-1) for p in model.parameters()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref)
    gflat = w.grad.value.clone()
    gref = gflat.clone()
    dist.broadcast(gref, src=0)
    assert torch.equal(gflat, gref)


def test_fp8_ddp_mnist_shaped_cnn_gloo():
    run_workers(_ddp_training, 2)


def _full_shard(rank, world):
    from msamp.fsdp import FP8FullyShardedDataParallel, FsdpReplacer
    torch.manual_seed(0)
    model = _mk_model()
    ref = _mk_model()
    fsdp = FP8FullyShardedDataParallel(model)
    assert len(fsdp.sharded) == 3 and fsdp.sharded[0].weight_shard.shape == (32 // world, 16)
    opt = fsdp.build_optimizer(torch.optim.AdamW, lr=1e-2)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2)
    x_all, y_all = torch.randn(8 * world, 16), torch.randn(8 * world, 4)
    for _ in range(10):
        xb, yb = x_all[rank * 8:(rank + 1) * 8], y_all[rank * 8:(rank + 1) * 8]
        loss = ((fsdp(xb) - yb)**2).mean()
        loss.backward()
        fsdp.step(opt, clip_grad=100.0)    # far above the norm: exercises the code without changing the comparison
        ropt.zero_grad()
        rl = ((ref(x_all) - y_all)**2).mean()
        rl.backward()
        ropt.step()
    full = ((fsdp(x_all) - y_all)**2).mean()
    assert abs(full.item() - ((ref(x_all) - y_all)**2).mean().item()) < 0.15 * rl.item() + 0.02
    # one scale per tensor on every shard
    s = fsdp.sharded[0].weight_meta.scale.clone()
    s2 = s.clone()
    dist.broadcast(s2, src=0)
    assert torch.equal(s, s2)
    # replicated (high-precision) parameters stay replicas
    hp = torch.cat([p.detach().float().reshape(-1) for p in fsdp.hp_params])
    hp2 = hp.clone()
    dist.broadcast(hp2, src=0)
    assert torch.equal(hp, hp2)
    # the torch-FSDP preparation path: fp32-viewed parameters carrying their meta
    from msamp.nn import model_state
    model_state.clear()
    m2 = FsdpReplacer.replace(_mk_model())
    p = m2[0].weight
    assert p.dtype == torch.float32 and p._original_shape == (32, 16) and p._padded == 0 and p._meta.qtype == E4M3
    out = m2(torch.randn(4, 16))
    out.sum().backward()
    assert p.grad is not None and p.grad.shape == p.shape


def test_full_shard_gloo():
    run_workers(_full_shard, 2)


def _torch_fsdp_fp8(rank, world):
    """FP8 weights inside torch's own FSDP (public hooks only): bytes are sharded, gradients reduced as FP8."""
    from msamp.fsdp.torch_fsdp import wrap_with_torch_fsdp
    from msamp.nn import model_state
    from msamp.optim import FSDPAdamW
    model_state.clear()
    torch.manual_seed(0)
    model = _mk_model()
    fsdp = wrap_with_torch_fsdp(model, device_id=torch.device('cpu'))
    params = list(fsdp.parameters())
    assert sum(hasattr(p, '_meta') for p in params) == 3    # the three linear weights carry FP8 bytes
    opt = FSDPAdamW(params, lr=1e-2, weight_decay=0.0)
    torch.manual_seed(5)
    x_all, y_all = torch.randn(8 * world, 16), torch.randn(8 * world, 4)
    losses = []
    for _ in range(12):
        xb, yb = x_all[rank * 8:(rank + 1) * 8], y_all[rank * 8:(rank + 1) * 8]
        loss = ((fsdp(xb) - yb)**2).mean()
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        losses.append(loss.item())
    assert losses[-1] < 0.9 * losses[0], losses
    # all shards of one weight share a scale
    for p in params:
        if hasattr(p, '_meta'):
            s = p._meta.scale.clone()
            ref = s.clone()
            dist.broadcast(ref, src=0)
            assert torch.equal(s, ref)


def test_torch_fsdp_with_fp8_weights_gloo():
    run_workers(_torch_fsdp_fp8, 2)


def _elastic_save(rank, world, path):
    torch.manual_seed(0)
    x_all, y_all = torch.randn(8 * world, 16), torch.randn(8 * world, 4)
    model = _mk_model()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    model, opt = msamp.initialize(model, opt, 'O2')
    zero = ZeroShardedOptimizer(model, opt, stage=2)
    for _ in range(5):
        loss = ((model(x_all[rank * 8:(rank + 1) * 8]) - y_all[rank * 8:(rank + 1) * 8])**2).mean()
        loss.backward()
        zero.reduce_and_step()
        for p in zero.hp_params:
            p.grad = None
    states = [None] * world
    dist.all_gather_object(states, zero.elastic_state_dict())
    if rank == 0:
        full = ZeroShardedOptimizer.consolidate_elastic_state(states)
        weights = [p.float() for p in zero.fp8_params]
        hp = [p.detach().clone() for p in zero.hp_params]
        torch.save({'opt': full, 'weights': weights, 'hp': hp}, path)


def _elastic_load(rank, world, path):
    ck = torch.load(path, weights_only=False)
    torch.manual_seed(123)    # a differently initialised model: everything must come from the checkpoint
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 32), torch.nn.GELU(), torch.nn.Linear(32, 4))
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    model, opt = msamp.initialize(model, opt, 'O2')
    zero = ZeroShardedOptimizer(model, opt, stage=2)
    with torch.no_grad():
        for p, saved in zip(zero.hp_params, ck['hp']):
            p.copy_(saved)
    zero.load_elastic_state_dict(ck['opt'])
    for p, want in zip(zero.fp8_params, ck['weights']):
        assert (p.float() - want).abs().max().item() <= 1e-6 + 0.07 * want.abs().max().item() / 8    # same e4m3 numbers
    for i, master in zero.masters.items():
        st = zero.optimizer.state[master]
        assert st['step'] == 5 and torch.equal(st['exp_avg'].value, ck['opt']['fp8'][i]['state']['exp_avg'].value)
    owned = sum(1 for o in zero.owners if o == rank)
    assert len(zero.masters) == owned
    # training goes on
    torch.manual_seed(0)
    x, y = torch.randn(8, 16), torch.randn(8, 4)
    loss = ((model(x) - y)**2).mean()
    loss.backward()
    zero.reduce_and_step()
    assert torch.isfinite(loss)
    assert all(zero.optimizer.state[m]['step'] == 6 for m in zero.masters.values())


def test_elastic_resume_at_another_degree(tmp_path):
    path = str(tmp_path / 'elastic.pt')
    run_workers(_elastic_save, 2, args=(path, ))
    run_workers(_elastic_load, 3, args=(path, ))
    run_workers(_elastic_load, 1, args=(path, ))


def _accumulation(rank, world, stage):
    """Two micro-batches in one step track one step on the concatenated batch."""
    from msamp.parallel import DataParallelTrainer

    class _Loss(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m

        def forward(self, x, y):
            return ((self.m(x) - y)**2).mean()

    def make():
        model = _mk_model()
        opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
        model, opt = msamp.initialize(model, opt, 'O2')
        return model, DataParallelTrainer(_Loss(model), opt, zero_stage=stage)

    torch.manual_seed(7)
    x_all, y_all = torch.randn(16 * world, 16), torch.randn(16 * world, 4)
    xs, ys = x_all[rank * 16:(rank + 1) * 16], y_all[rank * 16:(rank + 1) * 16]
    m1, t1 = make()
    from msamp.nn import model_state
    l1 = [t1.step(xs, ys).item() for _ in range(6)]
    model_state.clear()
    m2, t2 = make()
    l2 = [t2.step_micro_batches([(xs[:8], ys[:8]), (xs[8:], ys[8:])]).item() for _ in range(6)]
    assert l2[-1] < l2[0]
    assert max(abs(a - b) for a, b in zip(l1, l2)) < 0.05 * l1[0], (l1, l2)


def test_gradient_accumulation_trainer_ddp_and_zero2():
    run_workers(_accumulation, 2, args=(0, ))
    run_workers(_accumulation, 2, args=(2, ))


def _te_layer_zero2(rank, world):
    """Transformer-Engine-shaped layer under the sharded optimizer: two ranks end with identical weights."""
    from msamp.parallel import DataParallelTrainer
    from msamp.te import MSAMPTransformerLayer

    class _Loss(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layer = MSAMPTransformerLayer(64, 128, 4)

        def forward(self, x, y):
            return ((self.layer(x) - y)**2).mean()

    torch.manual_seed(0)
    net = _Loss()
    net, opt = msamp.initialize(net, None, 'O2', use_te=True)
    trainer = DataParallelTrainer(net, opt, zero_stage=2, clip_grad=1.0)
    torch.manual_seed(20 + rank)
    x, y = torch.randn(8, 4, 64), torch.randn(8, 4, 64)
    losses = [trainer.step(x, y).item() for _ in range(8)]
    assert losses[-1] < losses[0]
    flat = torch.cat([p.float().reshape(-1) for p in net.parameters()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref), (flat - ref).abs().max()


def test_te_transformer_layer_under_zero2():
    run_workers(_te_layer_zero2, 2)


def _ddp_accumulation_no_sync(rank, world):
    """FP8 DDP: two micro-batches with no_sync around the first equal one pass on the concatenated batch (closely)."""
    from msamp.nn import model_state

    def train(split):
        model_state.clear()
        torch.manual_seed(0)
        model = _mk_model()
        opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
        model, opt = msamp.initialize(model, opt, 'O2')
        ddp = torch.nn.parallel.DistributedDataParallel(model)
        torch.manual_seed(11 + rank)
        x, y = torch.randn(16, 16), torch.randn(16, 4)
        for _ in range(5):
            opt.zero_grad()
            if split:
                with ddp.no_sync():
                    (((ddp(x[:8]) - y[:8])**2).mean() / 2).backward()
                (((ddp(x[8:]) - y[8:])**2).mean() / 2).backward()
            else:
                ((ddp(x) - y)**2).mean().backward()
            opt.step()
        flat = torch.cat([p.float().reshape(-1) for p in model.parameters()])
        ref = flat.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(flat, ref), (flat - ref).abs().max()
        return flat

    a = train(False)
    b = train(True)
    # Adam turns tiny gradient differences (FP8 rounding of the accumulated gradient) into full-size steps for single
    # elements, so the comparison is on the average
    assert (a - b).abs().mean().item() < 0.02 * a.abs().mean().item(), ((a - b).abs().mean().item(), a.abs().mean().item())


def test_fp8_ddp_no_sync_accumulation():
    run_workers(_ddp_accumulation_no_sync, 2)


def _moe_local_params(rank, world, stage):
    """Expert parameters (``allreduce = False``) stay local: not averaged over the data-parallel group, their gradient
    norm is summed over it, and every rank clips with the same coefficient."""
    import msamp
    from msamp.deepspeed.runtime.fp8.fused_optimizer import FP8Optimizer
    torch.manual_seed(0)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.shared = torch.nn.Linear(8, 8)
            self.expert = torch.nn.Parameter(torch.full((8, ), float(rank + 1)))
            self.expert.allreduce = False

        def forward(self, x):
            return (self.shared(x) * self.expert).sum()

    model = Net()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    model, opt = msamp.initialize(model, opt, 'O2')
    fp8_opt = FP8Optimizer(model, opt, clip_grad=0.5, zero_stage=stage, fp8_master=stage > 0)
    if fp8_opt.zero is None:
        from msamp.parallel.zero import ZeroShardedOptimizer
        fp8_opt.zero = ZeroShardedOptimizer(model, opt, stage=0)
    assert [id(p) for p in fp8_opt.zero.local_params] == [id(model.expert)]
    x = torch.randn(4, 8)
    fp8_opt.backward(model(x))
    expert_grad = model.expert.grad.clone()
    fp8_opt.step()
    norms = [torch.zeros(()) for _ in range(world)]
    dist.all_gather(norms, fp8_opt.get_global_grad_norm().float().reshape(()))
    assert all(torch.equal(n, norms[0]) for n in norms)    # one norm for the whole job
    sq = expert_grad.square().sum().reshape(1)
    dist.all_reduce(sq)
    assert norms[0].item()**2 >= sq.item() * 0.999    # the expert part counts every rank's experts
    vals = [torch.zeros(8) for _ in range(world)]
    dist.all_gather(vals, model.expert.detach().clone())
    assert not torch.equal(vals[0], vals[1])    # experts were neither averaged nor broadcast


@pytest.mark.parametrize('stage', [0, 2])
def test_moe_expert_params_stay_local(stage):
    run_workers(_moe_local_params, 2, args=(stage, ))
