"""Megatron-style tensor/sequence parallel linears, local FP8 DDP and the distributed optimizer on gloo ranks."""
import math
import os
import tempfile

import torch
import torch.distributed as dist

from tests.dist_utils import run_workers


def _tp_block(rank, world, sequence_parallel):
    from msamp.megatron import ColumnParallelLinear, RowParallelLinear, parallel_state as mpu
    mpu.initialize_model_parallel(tensor_model_parallel_size=world)
    torch.manual_seed(0)
    H, F, S = 32, 64, 16
    full_w1 = torch.randn(F, H) * 0.1
    full_w2 = torch.randn(H, F) * 0.1
    x_full = torch.randn(S, 2, H)
    col = ColumnParallelLinear(H, F, bias=True, sequence_parallel=sequence_parallel)
    row = RowParallelLinear(F, H, bias=True, sequence_parallel=sequence_parallel)
    fs, hs = F // world, H
    with torch.no_grad():
        col.weight.copy_(full_w1[rank * fs:(rank + 1) * fs].cast(col.weight.qtype))
        row.weight.copy_(full_w2[:, rank * fs:(rank + 1) * fs].contiguous().cast(row.weight.qtype))
    x = x_full[rank * (S // world):(rank + 1) * (S // world)] if sequence_parallel else x_full
    x = x.clone().requires_grad_()
    y = row(torch.nn.functional.gelu(col(x)))
    ref_x = x_full.clone().requires_grad_()
    ref = torch.nn.functional.gelu(ref_x @ full_w1.t()) @ full_w2.t()
    want = ref[rank * (S // world):(rank + 1) * (S // world)] if sequence_parallel else ref
    assert y.shape == want.shape
    assert (y - want).abs().max() < 0.08, (y - want).abs().max()
    g_full = torch.randn(S, 2, H)
    g = g_full[rank * (S // world):(rank + 1) * (S // world)] if sequence_parallel else g_full
    y.backward(g)
    ref.backward(g_full)
    want_dx = ref_x.grad[rank * (S // world):(rank + 1) * (S // world)] if sequence_parallel else ref_x.grad
    assert (x.grad - want_dx).abs().max() < 0.2 * want_dx.abs().max() + 0.05    # two chained GEMMs with e5m2 gradients
    gw1 = col.weight.grad
    # weight gradients against autograd of the dense reference
    w1 = full_w1.clone().requires_grad_()
    w2 = full_w2.clone().requires_grad_()
    (torch.nn.functional.gelu(x_full @ w1.t()) @ w2.t()).backward(g_full)
    got1 = gw1.float() if hasattr(gw1, 'meta') and not torch.is_tensor(gw1) else gw1
    got2 = row.weight.grad
    got2 = got2.float() if not torch.is_tensor(got2) else got2
    assert (got1 - w1.grad[rank * fs:(rank + 1) * fs]).abs().max() < 0.12 * w1.grad.abs().max()
    assert (got2 - w2.grad[:, rank * fs:(rank + 1) * fs]).abs().max() < 0.12 * w2.grad.abs().max()
    mpu.destroy_model_parallel()


def test_tensor_parallel_block_allreduce():
    run_workers(_tp_block, 2, args=(False, ))


def test_sequence_parallel_block():
    run_workers(_tp_block, 2, args=(True, ))


def _ddp_distopt(rank, world):
    import msamp
    from msamp.megatron import FP8DistributedDataParallel, FP8DistributedOptimizer, clip_grad_norm_fp32, parallel_state as mpu
    from msamp.optim import LBAdamW
    mpu.initialize_model_parallel(tensor_model_parallel_size=1)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 32), torch.nn.GELU(), torch.nn.Linear(32, 4))
    model = msamp.nn.LinearReplacer.replace(model)
    ddp = FP8DistributedDataParallel(model, accumulate_allreduce_grads_in_fp32=True, use_contiguous_buffers=True)
    assert sum(b - a for a, b in ddp.fp8_partitions) == sum(p.numel() for p in ddp.fp8_params)
    opt = FP8DistributedOptimizer(LBAdamW(model.parameters(), lr=1e-2), clip_grad=1.0, models=[ddp])
    x_all, y_all = torch.randn(16 * world, 16), torch.randn(16 * world, 4)
    losses = []
    for it in range(10):
        opt.zero_grad()
        for micro in range(2):    # two micro-batches accumulate into the FP8 main grads
            lo = rank * 16 + micro * 8
            loss = ((ddp(x_all[lo:lo + 8]) - y_all[lo:lo + 8])**2).mean() / 2
            loss.backward()
        opt.reduce_model_grads()
        ok, norm, _ = opt.step()
        assert ok and norm is not None and norm > 0
        losses.append(loss.item())
    assert losses[-1] < losses[0]
    flat = torch.cat([p.float().reshape(-1) for p in model.parameters()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref)
    sd = opt.state_dict()
    assert 'param_groups' in sd['optimizer'] and 'params' not in sd['optimizer']['param_groups'][0]
    path = os.path.join(tempfile.gettempdir(), 'msamp_distrib_opt_test.pt')
    opt.save_parameter_state(path)
    dist.barrier()
    before = flat.clone()
    opt.load_parameter_state(path)
    after = torch.cat([p.float().reshape(-1) for p in model.parameters()])
    assert (before - after).abs().max() < 0.05 * before.abs().max()
    st = torch.load(path, weights_only=False)
    assert set(st[0].keys()) == {torch.uint8, torch.float32} and set(st[0][torch.uint8]) == {'param', 'exp_avg', 'exp_avg_sq'}
    assert clip_grad_norm_fp32([torch.nn.Parameter(torch.ones(4))], [torch.ones(4) * 3], 1.0) == 6.0
    mpu.destroy_model_parallel()


def test_local_ddp_and_distributed_optimizer():
    run_workers(_ddp_distopt, 2)


def _parallel_gpt(rank, world, tp, sp=True):
    import msamp
    from msamp.megatron import parallel_state as mpu
    from msamp.models import GPT, ParallelGPT, gpt_config
    from msamp.optim import LBAdamW
    from msamp.parallel import DataParallelTrainer
    mpu.initialize_model_parallel(tensor_model_parallel_size=tp)
    dp_rank = mpu.get_data_parallel_rank()
    cfg = gpt_config('gpt-tiny', n_layer=2, n_head=4, hidden=64, ffn_hidden=256, vocab_size=128, max_seq=32)
    torch.manual_seed(0)
    model = ParallelGPT(cfg, act_dtype=torch.float32, sequence_parallel=sp)
    assert model.sequence_parallel == (sp and tp > 1)
    opt = LBAdamW(model.parameters(), lr=3e-3)
    trainer = DataParallelTrainer(model, opt, zero_stage=2 if world > tp else 0, group=mpu.get_data_parallel_group(),
                                  after_backward=model.allreduce_sequence_parallel_grads, clip_grad=0.5,
                                  model_parallel_group=mpu.get_model_parallel_group())
    torch.manual_seed(100 + dp_rank)    # same data inside a tensor-parallel group
    tok = torch.randint(0, cfg.vocab_size, (2, 16))
    losses = [trainer.step(tok, tok).item() for _ in range(12)]
    assert losses[-1] < losses[0] - 0.2, losses
    assert abs(losses[0] - math.log(cfg.vocab_size)) < 0.5
    # the loss is a property of the tensor-parallel group, replicated parameters stay replicas
    t = torch.tensor(losses)
    ref = t.clone()
    dist.broadcast(ref, src=mpu.get_tensor_model_parallel_src_rank(), group=mpu.get_tensor_model_parallel_group())
    assert torch.allclose(t, ref, atol=1e-5)
    flat = torch.cat([p.detach().float().reshape(-1) for p in model.replicated_parameters()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.allclose(flat, ref, atol=1e-6)
    mpu.destroy_model_parallel()


def test_parallel_gpt_tp2_sequence_parallel():
    run_workers(_parallel_gpt, world=2, backend='gloo', args=(2, ))


def test_parallel_gpt_tp2_dp2():
    run_workers(_parallel_gpt, world=4, backend='gloo', args=(2, ))


def _vocab_parallel_xent(rank, world):
    from msamp.megatron import parallel_state as mpu
    from msamp.models import vocab_parallel_cross_entropy
    mpu.initialize_model_parallel(tensor_model_parallel_size=world)
    torch.manual_seed(3)
    full = torch.randn(24, 40)
    labels = torch.randint(0, 40, (24, ))
    ref_in = full.clone().requires_grad_()
    ref = torch.nn.functional.cross_entropy(ref_in, labels)
    ref.backward()
    v = 40 // world
    mine = full[:, rank * v:(rank + 1) * v].clone().requires_grad_()
    loss = vocab_parallel_cross_entropy(mine, labels, rank * v)
    loss.backward()
    assert torch.allclose(loss, ref, atol=1e-5)
    assert torch.allclose(mine.grad, ref_in.grad[:, rank * v:(rank + 1) * v], atol=1e-6)
    mpu.destroy_model_parallel()


def test_vocab_parallel_cross_entropy_matches_torch():
    run_workers(_vocab_parallel_xent, world=2, backend='gloo')


def _parallel_gpt_distopt(rank, world, tp):
    """ParallelGPT under the Megatron-style FP8 DDP buffers + distributed optimizer (TP x DP)."""
    from msamp.megatron import FP8DistributedDataParallel, FP8DistributedOptimizer, parallel_state as mpu
    from msamp.models import ParallelGPT, gpt_config
    from msamp.optim import LBAdamW
    mpu.initialize_model_parallel(tensor_model_parallel_size=tp)
    cfg = gpt_config('gpt-tiny', n_layer=2, n_head=4, hidden=64, ffn_hidden=256, vocab_size=128, max_seq=32)
    torch.manual_seed(0)
    model = ParallelGPT(cfg, act_dtype=torch.float32)
    ddp = FP8DistributedDataParallel(model, accumulate_allreduce_grads_in_fp32=True, use_contiguous_buffers=True)
    opt = FP8DistributedOptimizer(LBAdamW(model.parameters(), lr=3e-3), clip_grad=1.0, models=[ddp])
    torch.manual_seed(100 + mpu.get_data_parallel_rank())
    tok = torch.randint(0, cfg.vocab_size, (2, 16))
    losses = []
    for _ in range(12):
        opt.zero_grad()
        loss = ddp(tok, tok)
        loss.backward()
        model.allreduce_sequence_parallel_grads()
        opt.reduce_model_grads()
        ok, norm, _ = opt.step()
        assert ok
        losses.append(loss.item())
    assert losses[-1] < losses[0] - 0.2, losses
    flat = torch.cat([p.detach().float().reshape(-1) for p in model.replicated_parameters()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.allclose(flat, ref, atol=1e-6)
    mpu.destroy_model_parallel()


def test_parallel_gpt_under_distributed_optimizer_tp2_dp2():
    run_workers(_parallel_gpt_distopt, world=4, backend='gloo', args=(2, ))


def _local_ddp_allreduce(rank, world):
    """Megatron-style local DDP with the replicated optimizer: allreduce_gradients + clip + LBAdamW keeps replicas equal."""
    import msamp
    from msamp.megatron import FP8DistributedDataParallel, clip_grad_norm_fp32, parallel_state as mpu
    from msamp.optim import LBAdamW
    mpu.initialize_model_parallel(tensor_model_parallel_size=1)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 4))
    model = msamp.nn.LinearReplacer.replace(model)
    ddp = FP8DistributedDataParallel(model, accumulate_allreduce_grads_in_fp32=True, use_contiguous_buffers=True)
    opt = LBAdamW(model.parameters(), lr=1e-2)
    torch.manual_seed(10)
    x_all, y_all = torch.randn(16 * world, 16), torch.randn(16 * world, 4) * 3
    first = last = None
    for it in range(12):
        ddp.zero_grad_buffer()
        for micro in range(2):
            lo = rank * 16 + micro * 8
            loss = ((ddp(x_all[lo:lo + 8]) - y_all[lo:lo + 8])**2).mean() / 2
            loss.backward()
        ddp.allreduce_gradients()
        params = list(model.parameters())
        for p in params:
            p.grad = p.main_grad
        clip_grad_norm_fp32(params, [p.grad for p in params], 1.0)
        opt.step()
        for p in params:
            p.grad = None
        full = ((ddp(x_all) - y_all)**2).mean().item()
        first = full if first is None else first
        last = full
    assert last < first
    flat = torch.cat([p.float().reshape(-1) for p in model.parameters()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref), (flat - ref).abs().max()
    mpu.destroy_model_parallel()


def test_local_ddp_allreduce_keeps_replicas_equal():
    run_workers(_local_ddp_allreduce, world=2, backend='gloo')


def test_parallel_gpt_tp4():
    run_workers(_parallel_gpt, world=4, backend='gloo', args=(4, ))


def test_parallel_gpt_tp2_without_sequence_parallel():
    run_workers(_parallel_gpt, world=2, backend='gloo', args=(2, False))


def _tp_matches_unsharded(rank, world):
    """The loss and an input-embedding gradient of ParallelGPT at tp=2 (sequence parallel) equal those of the same weights unsharded."""
    from msamp.common.dtype import Dtypes
    from msamp.megatron import parallel_state as mpu
    from msamp.models import ParallelGPT, gpt_config
    from msamp.nn import model_state
    cfg = gpt_config('gpt-tiny', n_layer=2, n_head=4, hidden=64, ffn_hidden=256, vocab_size=128, max_seq=32)
    mpu.initialize_model_parallel(tensor_model_parallel_size=2)
    tp_group = mpu.get_tensor_model_parallel_group()
    torch.manual_seed(0)
    sharded = ParallelGPT(cfg, act_dtype=torch.float32)
    torch.manual_seed(7)
    tok = torch.randint(0, cfg.vocab_size, (2, 16))
    loss_tp = sharded(tok, tok)
    loss_tp.backward()
    sharded.allreduce_sequence_parallel_grads()
    g_tp = sharded.wpe.weight.grad.clone()

    def gather(t, dim):
        parts = [torch.empty_like(t) for _ in range(2)]
        dist.all_gather(parts, t.contiguous(), group=tp_group)
        return parts if dim is None else torch.cat(parts, dim)

    full = {}
    for name, p in sharded.named_parameters():
        v = p.float() if hasattr(p, 'meta') else p.detach()
        if name.endswith('qkv.weight') or name.endswith('qkv.bias'):
            parts = gather(v, None)    # each [3 * hl * d, ...] laid out (3, hl, d)
            hl, d = cfg.n_head // 2, cfg.head_dim
            stacked = torch.stack([q.reshape(3, hl, d, *q.shape[1:]) for q in parts], dim=1)    # [3, tp, hl, d, ...]
            full[name] = stacked.reshape(3 * cfg.n_head * d, *v.shape[1:])
        elif any(name.endswith(k) for k in ('fc1.weight', 'fc1.bias', 'lm_head.weight')):
            full[name] = gather(v, 0)
        elif any(name.endswith(k) for k in ('proj.weight', 'fc2.weight')):
            full[name] = gather(v, 1)
        else:
            full[name] = v.clone()
    mpu.destroy_model_parallel()
    model_state.clear()
    mpu.initialize_model_parallel(tensor_model_parallel_size=1)
    whole = ParallelGPT(cfg, act_dtype=torch.float32)
    with torch.no_grad():
        for name, p in whole.named_parameters():
            if hasattr(p, 'meta'):
                p.copy_(full[name].cast(Dtypes.kfloat16))
            else:
                p.copy_(full[name])
    loss_1 = whole(tok, tok)
    loss_1.backward()
    assert abs(loss_tp.item() - loss_1.item()) < 2e-3 * abs(loss_1.item()), (loss_tp.item(), loss_1.item())
    g_1 = whole.wpe.weight.grad
    assert (g_tp - g_1).abs().max().item() < 0.05 * g_1.abs().max().item() + 1e-5
    mpu.destroy_model_parallel()


def test_tensor_parallel_gpt_matches_unsharded_weights():
    run_workers(_tp_matches_unsharded, world=2, backend='gloo')


def test_parallel_gpt_state_dict_roundtrip(tmp_path):
    """ScalingParameters of the parallel linears survive torch.save / load_state_dict (single rank, tp = 1)."""
    from msamp.megatron import parallel_state as mpu
    from msamp.models import ParallelGPT, gpt_config
    from msamp.nn import model_state
    mpu.initialize_model_parallel(tensor_model_parallel_size=1)
    cfg = gpt_config('gpt-tiny', n_layer=1, n_head=2, hidden=32, ffn_hidden=64, vocab_size=64, max_seq=16)
    torch.manual_seed(0)
    a = ParallelGPT(cfg, act_dtype=torch.float32)
    tok = torch.randint(0, 64, (2, 16))
    want = a(tok, tok).item()
    path = str(tmp_path / 'pgpt.pt')
    torch.save(a.state_dict(), path)
    model_state.clear()
    torch.manual_seed(5)
    b = ParallelGPT(cfg, act_dtype=torch.float32)
    assert abs(b(tok, tok).item() - want) > 1e-4
    b.load_state_dict(torch.load(path, weights_only=False))
    assert abs(b(tok, tok).item() - want) < 1e-6
    mpu.destroy_model_parallel()
