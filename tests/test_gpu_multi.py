"""Multi-GPU tests: symmetric memory, fused FP8 reduce, sharded optimizer, fused GEMM + collective kernels.

Every test runs on 2, 4 and 8 ranks (one process per GPU) and is skipped when fewer GPUs are visible."""
import os

import pytest
import torch
import torch.distributed as dist

import msamp
from msamp.common.dtype import Dtypes
from tests.dist_utils import run_workers

pytestmark = pytest.mark.gpu
E4M3 = Dtypes.kfloat8_e4m3
# MSAMP_TEST_WORLDS narrows the rank counts (a box with eight GPUs is expensive: see test_all_scenarios_in_one_group)
WORLDS = pytest.mark.parametrize('world', [int(w) for w in os.getenv('MSAMP_TEST_WORLDS', '2,4,8').split(',') if w])


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
    # guard regions on either side of the buffer: intact after the writes above, and a changed byte is reported
    from msamp.parallel.symm import GuardCorruption
    buf.check_guards()
    flags.check_guards()
    after = buf._guard_views()[1]
    after[7] = 0    # host-injected: what an out-of-range store of a kernel would leave behind
    with pytest.raises(GuardCorruption):
        buf.check_guards()
    after[7] = buf.GUARD_BYTE
    buf.close()
    flags.close()


@WORLDS
def test_symmetric_memory_and_bounded_barrier(world):
    _need(world)
    run_workers(_symm_and_barrier, world, backend='nccl')


def _timeout_then_normal_reduce(rank, world):
    """Host-injected failure of the fused gradient reduce: the ranks disagree on the epoch, so one side's wait runs out
    (status bit 1) and the other sees a flag from the future (status bit 3); after the ranks agree again the very next
    reduce must be correct, i.e. the shared completion counter was left at zero by the CTAs that gave up."""
    from msamp.ops import native
    from msamp.parallel.zero import ZeroShardedOptimizer
    dev = torch.device('cuda', rank)
    model = _mk_model(dev)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    model, opt = msamp.initialize(model, opt, 'O2')
    zero = ZeroShardedOptimizer(model, opt, stage=0, wait_seconds=1.0)
    torch.manual_seed(100 + rank)
    x = torch.randn(64, 256, device=dev)
    model(x).square().mean().backward()
    keep = zero.g_flat.clone()
    keep_meta = zero.g_meta_t.clone()
    if rank == 0:
        zero.flags.epoch += 100    # rank 0 waits for an epoch nobody else announces
    zero._reduce_fp8_grads()
    torch.cuda.synchronize()
    status = native.device_status()
    assert status & (2 if rank == 0 else 8), status
    counter = zero.flags.view(torch.int32)[-8:]
    assert int(counter[0]) == 0    # the completion counter is back at zero
    # agree on the epoch again (on the host) and restore the inputs: the next reduce is a normal one
    dist.barrier()
    zero.flags.epoch = 1000
    zero.g_flat.copy_(keep)
    zero.g_meta_t.copy_(keep_meta)
    torch.cuda.synchronize()
    dist.barrier()
    expect = []
    for i, p in enumerate(zero.fp8_params):
        lo = zero.offsets[i]
        g = keep[lo:lo + p.numel()].view(torch.float8_e4m3fn).float() * keep_meta[0, i]
        dist.all_reduce(g)
        expect.append(g / world)
    zero._reduce_fp8_grads()
    torch.cuda.synchronize()
    assert native.device_status() == 0
    for i, (p, e) in enumerate(zip(zero.fp8_params, expect)):
        lo = zero.offsets[i]
        got = zero.g_flat[lo:lo + p.numel()].view(torch.float8_e4m3fn).float() * zero.g_meta_t[0, i]
        assert (got - e).abs().max().item() <= 0.07 * e.abs().max().item() + 1e-8
    zero.close()


@WORLDS
def test_reduce_recovers_after_timeout_and_detects_desync(world):
    _need(world)
    run_workers(_timeout_then_normal_reduce, world, backend='nccl')


def _fp8_ddp_fused(rank, world):
    """FP8 DDP on the fused all-reduce kernel: the reduced gradient is the fp32 mean of the ranks' gradients within one
    e4m3 rounding, every rank ends with identical bytes and scales, and training converges with identical replicas."""
    from msamp.nn.distributed import FP8DistributedDataParallel
    from msamp.ops import native
    dev = torch.device('cuda', rank)
    model = _mk_model(dev)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    model, opt = msamp.initialize(model, opt, 'O2')
    ddp = FP8DistributedDataParallel(model, device_ids=[rank], bucket_cap_mb=0.2)
    red = ddp.scaling_tensor_reducer
    assert red.fused and len(red.bucket_to_param_ids) > 1
    torch.manual_seed(50 + rank)
    x = torch.randn(64, 256, device=dev)
    ddp(x).square().mean().backward()
    torch.cuda.synchronize()
    assert native.device_status() == 0
    for p in red.parameters:
        assert p.grad is not None and p.grad.qtype == E4M3
    flat = red.g_flat.clone()
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref)
    meta = red.g_meta_t[0].clone()
    ref = meta.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(meta, ref)
    opt.zero_grad()
    xs, ys = torch.randn(world * 32, 256, device=dev), torch.randn(world * 32, 64, device=dev)
    dist.broadcast(xs, src=0)
    dist.broadcast(ys, src=0)
    losses = []
    for _ in range(20):
        opt.zero_grad()
        loss = (ddp(xs[rank * 32:(rank + 1) * 32]) - ys[rank * 32:(rank + 1) * 32]).square().mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    torch.cuda.synchronize()
    assert native.device_status() == 0
    assert losses[-1] < 0.8 * losses[0], losses
    flat = torch.cat([p.float().reshape(-1) for p in model.parameters()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref)
    red.close()


@WORLDS
def test_fp8_ddp_on_fused_allreduce(world):
    _need(world)
    run_workers(_fp8_ddp_fused, world, backend='nccl')


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
    zero.close()    # also checks the guard regions around the symmetric buffers


@WORLDS
def test_fused_fp8_allreduce(world):
    _need(world)
    run_workers(_fused_reduce_matches_math, world, backend='nccl')


def _zero2_training(rank, world, fuse_adam=True, overlap=False):
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
    trainer = DataParallelTrainer(wrapped, opt, zero_stage=2, overlap_comm=overlap)
    if overlap:
        assert trainer.zero.overlap_comm
        assert len(trainer.zero.buckets) >= 1
    trainer.zero.fuse_adam = trainer.zero.fuse_adam and fuse_adam
    assert trainer.zero.fuse_adam == fuse_adam
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
    trainer.zero.close()


def _fused_adam_equals_reduce_then_adam(rank, world):
    """One optimizer step from the same gradients and states, once with the reduce-scatter folded into the Adam kernel and
    once with the separate reduce kernel: masters, moments and published FP8 weights agree bit for bit."""
    from msamp.ops import native
    from msamp.parallel.zero import ZeroShardedOptimizer
    dev = torch.device('cuda', rank)
    model = _mk_model(dev)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    model, opt = msamp.initialize(model, opt, 'O2')
    zero = ZeroShardedOptimizer(model, opt, stage=2)
    assert zero.fuse_adam
    torch.manual_seed(100 + rank)
    x = torch.randn(64, 256, device=dev)
    model(x).square().mean().backward()
    torch.cuda.synchronize()
    dist.barrier()
    snap = dict(g=zero.g_flat.clone(), gm=zero.g_meta_t.clone(), w=zero.w_flat.clone(), wm=zero.w_meta_t.clone(),
                masters={i: (m.value.clone(), m.meta.scale.clone(), m.meta.scale_inv.clone(), m.meta.amax.clone()) for i, m in zero.masters.items()},
                hp=[p.detach().clone() for p in zero.hp_params], hp_grads=[None if p.grad is None else p.grad.clone() for p in zero.hp_params],
                fp8_grads=[p.grad for p in zero.fp8_params])
    results = []
    for fused in (True, False):
        zero.fuse_adam = fused
        zero.reduce_and_step()
        torch.cuda.synchronize()
        assert native.device_status() == 0
        dist.barrier()
        results.append(dict(w=zero.w_flat.clone(), wm=zero.w_meta_t[:2].clone(),
                            masters={i: m.value.clone() for i, m in zero.masters.items()},
                            m={i: opt.state[m]['exp_avg'].value.clone() for i, m in zero.masters.items()},
                            v={i: opt.state[m]['exp_avg_sq'].value.clone() for i, m in zero.masters.items()}))
        # back to the state before the step
        opt.state.clear()
        zero.g_flat.copy_(snap['g'])
        zero.g_meta_t.copy_(snap['gm'])
        zero.w_flat.copy_(snap['w'])
        zero.w_meta_t.copy_(snap['wm'])
        for i, m in zero.masters.items():
            val, sc, si, am = snap['masters'][i]
            m.value.copy_(val)
            m.meta.scale.copy_(sc)
            m.meta.scale_inv.copy_(si)
            m.meta.amax.copy_(am)
        for p, d, g in zip(zero.hp_params, snap['hp'], snap['hp_grads']):
            p.data.copy_(d)
            p.grad = None if g is None else g.clone()
        for p, g in zip(zero.fp8_params, snap['fp8_grads']):
            p.grad = g
        torch.cuda.synchronize()
        dist.barrier()
    a, b = results
    assert torch.equal(a['w'], b['w']) and torch.equal(a['wm'], b['wm'])
    for i in a['masters']:
        assert torch.equal(a['masters'][i], b['masters'][i]) and torch.equal(a['m'][i], b['m'][i]) and torch.equal(a['v'][i], b['v'][i])
    zero.close()


@WORLDS
def test_zero2_training(world):
    _need(world)
    run_workers(_zero2_training, world, backend='nccl', args=(True, ))


@WORLDS
def test_zero2_reduction_overlapped_with_backward(world):
    """The FP8 gradients are reduced bucket by bucket from backward hooks on a side stream; replicas agree, the loss falls."""
    _need(world)
    run_workers(_zero2_training, world, backend='nccl', args=(True, True))


@WORLDS
def test_reduce_scatter_fused_into_adam_is_bit_exact(world):
    _need(world)
    run_workers(_fused_adam_equals_reduce_then_adam, world, backend='nccl')


def _fused_gemms(rank, world, n_comm=4, shapes=((128, 256, 128), (256, 512, 384), (1024, 4096, 1536), (512, 1024, 1000))):
    from msamp.ops import cast, gemm, native
    from msamp.parallel.fused import FusedGemmContext, all_gather_cols, all_gather_rows, reduce_scatter_rows
    dev = torch.device('cuda', rank)
    F8 = Dtypes.qtype_to_float8
    ctx = FusedGemmContext(max_shard_bytes=8 << 20, max_out_bytes=64 << 20, n_comm=n_comm, wait_seconds=2.0)
    assert ctx.native
    sinv = torch.tensor(1 / 16.0, device=dev)
    scale = torch.tensor(16.0, device=dev)

    def q(shape, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        return cast.cast_to_fp8(torch.randn(*shape, device=dev, generator=g), E4M3, scale)

    for (rows, K, N) in shapes:
        # --- all-gather(rows of A) + GEMM
        a_shard = q((rows, K), 100 + rank)
        b = q((N, K), 7)
        view = ctx.shard_view(rows * K).view(rows, K)
        view.copy_(a_shard)
        bias = torch.randn(N, device=dev)
        out = ctx.ag_rows_gemm(view, E4M3, sinv, b, E4M3, sinv, torch.bfloat16, bias=bias)
        full = all_gather_rows(a_shard)
        ref = gemm.gemm_fp8(full, E4M3, sinv, b, E4M3, sinv, torch.bfloat16, bias=bias)
        torch.cuda.synchronize()
        assert native.device_status() == 0
        assert torch.equal(out, ref), ('ag_rows a', rows, K, N, (out.float() - ref.float()).abs().max().item())
        assert torch.equal(ctx.gathered_rows(rows, K), full)
        # --- all-gather(rows of B) + GEMM (parameter gather); 384 = 3 x 128 rows per shard forces the 128 x 128 tiles
        # (a 256-row tile would straddle two ranks' shards), as the 896- and 2688-row shards of a 7168-wide model do
        for w_rows in (256, 384):
            w_shard = q((w_rows, K), 200 + rank)
            x = q((rows, K), 9)
            view = ctx.shard_view(w_rows * K).view(w_rows, K)
            view.copy_(w_shard)
            out = ctx.ag_rows_gemm(view, E4M3, sinv, x, E4M3, sinv, torch.bfloat16, shard_is='b')
            ref = gemm.gemm_fp8(x, E4M3, sinv, all_gather_rows(w_shard), E4M3, sinv, torch.bfloat16)
            torch.cuda.synchronize()
            assert native.device_status() == 0
            assert torch.equal(out, ref), ('ag_rows b', rows, K, w_rows)
        # --- GEMM with K-gathered B (wgrad shape): D[N, K] = A[N, W*rows] . concat_K(B_r[K, rows])^T
        a_full = q((N, rows * world), 11)
        bt_shard = q((K, rows), 300 + rank)
        if rows % 128 == 0:
            view = ctx.shard_view(((K + 255) // 256 * 256) * rows)[:K * rows].view(K, rows)
            view.copy_(bt_shard)
            am = torch.zeros((), device=dev)
            out = ctx.ag_k_gemm(a_full, E4M3, sinv, view, E4M3, sinv, torch.float32, amax_out=am)
            ref = gemm.gemm_fp8(a_full, E4M3, sinv, all_gather_cols(bt_shard), E4M3, sinv, torch.float32)
            torch.cuda.synchronize()
            assert native.device_status() == 0
            err = (out - ref).abs().max().item()
            assert err <= 1e-3 * ref.abs().max().item() + 1e-4, ('ag_k', rows, K, N, err)    # summation order differs
            assert abs(am.item() - out.abs().max().item()) <= 1e-6 * am.item() + 1e-6
        # --- GEMM + reduce-scatter
        M = rows * world
        a_part = q((M, K), 400 + rank)
        b_part = q((N, K), 500 + rank)
        if (N * 2) % 16 == 0:
            out = ctx.gemm_rs(a_part, E4M3, sinv, b_part, E4M3, sinv, torch.bfloat16)
            part = gemm.gemm_fp8(a_part, E4M3, sinv, b_part, E4M3, sinv, torch.float32)
            ref = reduce_scatter_rows(part)
            torch.cuda.synchronize()
            assert native.device_status() == 0
            err = (out.float() - ref).abs().max().item()
            assert err <= 2e-2 * ref.abs().max().item() + 1e-3, ('gemm_rs', rows, K, N, err)    # partials are rounded to bf16 before the sum
    dist.barrier()
    ctx.close()


@WORLDS
def test_fused_gemm_collectives(world):
    _need(world)
    run_workers(_fused_gemms, world, backend='nccl')


@pytest.mark.parametrize('n_comm', [1, 32])
def test_fused_gemm_copy_cta_extremes(n_comm):
    """One copy CTA (every chunk through the same CTA) and many (more copy CTAs than chunks for the small shapes)."""
    _need(2)
    run_workers(_fused_gemms, 2, backend='nccl', args=(n_comm, ((128, 256, 128), (512, 1024, 1000))))


def _skewed(rank, world):
    from msamp.parallel import symm
    assert symm._SKEW_US == 300.0
    _fused_reduce_matches_math(rank, world)
    _fused_gemms(rank, world, 4, ((128, 256, 128), (512, 1024, 1000)))
    _fused_adam_equals_reduce_then_adam(rank, world)


@pytest.mark.parametrize('order', ['forward', 'reverse'])
def test_rank_skewed_schedules(order, monkeypatch):
    """The cross-rank kernels under two deterministic, opposite arrival orders (rank r enters every cross-rank launch
    300 us x r late, or 300 us x (world - 1 - r) late)."""
    world = 4 if torch.cuda.is_available() and torch.cuda.device_count() >= 4 else 2
    _need(world)
    monkeypatch.setenv('MSAMP_DEBUG_SKEW_US', '300')
    monkeypatch.setenv('MSAMP_DEBUG_SKEW_ORDER', order)
    run_workers(_skewed, world, backend='nccl')


def _sp_block_fused(rank, world):
    """A sequence-parallel MLP block (column-parallel, GeLU, row-parallel) on the fused gather-GEMM / GEMM-reduce-scatter
    kernels against (a) the SAME FP8 computation composed of NCCL collectives and the plain GEMM, which it must match
    within the rounding of the bf16 partial sums, and (b) fp32 math, loosely (FP8 quantisation error)."""
    from msamp.megatron import ColumnParallelLinear, RowParallelLinear, layers, parallel_state as mpu
    from msamp.ops import native
    mpu.initialize_model_parallel(tensor_model_parallel_size=world)
    dev = torch.device('cuda', rank)
    torch.manual_seed(0)
    H, F, S, B = 256, 1024, 256 * world, 1
    full_w1 = (torch.randn(F, H, device=dev) * 0.05)
    full_w2 = (torch.randn(H, F, device=dev) * 0.05)
    x_full = torch.randn(S, B, H, device=dev)
    g_full = torch.randn(S, B, H, device=dev)
    fs = F // world
    sl = slice(rank * (S // world), (rank + 1) * (S // world))

    def run(fused):
        layers.USE_FUSED_COLLECTIVES = fused
        torch.manual_seed(1)
        col = ColumnParallelLinear(H, F, bias=True, sequence_parallel=True, device=dev)
        row = RowParallelLinear(F, H, bias=True, sequence_parallel=True, device=dev)
        with torch.no_grad():
            col.weight.copy_(full_w1[rank * fs:(rank + 1) * fs].cast(col.weight.qtype))
            row.weight.copy_(full_w2[:, rank * fs:(rank + 1) * fs].contiguous().cast(row.weight.qtype))
        x = x_full[sl].bfloat16().clone().requires_grad_()
        y = row(torch.nn.functional.gelu(col(x)))
        if fused:
            assert mpu.get_fused_context().native
        y.backward(g_full[sl].bfloat16())
        torch.cuda.synchronize()
        assert native.device_status() == 0
        return y.detach().float(), x.grad.float(), col.weight.grad.float(), row.weight.grad.float()

    try:
        fused = run(True)
        plain = run(False)
    finally:
        layers.USE_FUSED_COLLECTIVES = True
    # (a) same FP8 operands, same products: only the order / precision of the cross-rank sums differs (fp32 in the fused
    # epilogue, bf16 in NCCL), and a weight gradient may land on the other side of one e4m3 rounding boundary
    names = ('y', 'dx', 'wgrad_col', 'wgrad_row')
    tols = (0.02, 0.02, 0.07, 0.07)
    for name, a, b, tol in zip(names, fused, plain, tols):
        scale = b.abs().max().item()
        assert (a - b).abs().max().item() <= tol * scale + 1e-6, (name, (a - b).abs().max().item(), scale)
        if name.startswith('wgrad'):
            assert (a != b).float().mean().item() < 0.02, (name, (a != b).float().mean().item())
    # (b) fp32 math
    y, dx, wg1, wg2 = fused
    w1 = full_w1.clone().requires_grad_()
    w2 = full_w2.clone().requires_grad_()
    ref_x = x_full.clone().requires_grad_()
    ref = torch.nn.functional.gelu(ref_x @ w1.t()) @ w2.t()
    ref.backward(g_full)
    assert (y - ref[sl]).abs().max().item() < 0.1 * ref.abs().max().item() + 0.02    # two chained FP8 GEMMs
    assert (dx - ref_x.grad[sl]).abs().max().item() < 0.25 * ref_x.grad.abs().max().item()
    assert (wg1 - w1.grad[rank * fs:(rank + 1) * fs]).abs().max().item() < 0.15 * w1.grad.abs().max().item()
    assert (wg2 - w2.grad[:, rank * fs:(rank + 1) * fs]).abs().max().item() < 0.15 * w2.grad.abs().max().item()
    mpu.destroy_model_parallel()


@WORLDS
def test_sequence_parallel_block_fused_kernels(world):
    _need(world)
    run_workers(_sp_block_fused, world, backend='nccl')


def _full_shard_fused(rank, world):
    from msamp.fsdp import FP8FullyShardedDataParallel
    from msamp.ops import native
    dev = torch.device('cuda', rank)
    torch.manual_seed(0)
    # shards of 384 = 3 x 128 rows (not a multiple of the 256-row tile) and of 128 rows; an embedding-like parameter
    # that is not a linear gets an owner rank instead of being replicated
    hidden = 384 * world
    model = torch.nn.Sequential(torch.nn.Linear(512, hidden), torch.nn.GELU(), torch.nn.Linear(hidden, 128 * world)).to(dev)
    extra = torch.nn.Parameter(torch.zeros(128 * world, device=dev))
    model.register_parameter('out_shift', extra)
    fsdp = FP8FullyShardedDataParallel(model)
    assert fsdp.ctx is not None and fsdp.ctx.native and len(fsdp.sharded) == 2 and all(m.resident for m in fsdp.sharded)
    opt = fsdp.build_optimizer(torch.optim.AdamW, lr=2e-3)
    n_opt = sum(len(g['params']) for g in opt.param_groups)
    assert n_opt == 2 + len(fsdp.hp.owned()) < 2 + len(fsdp.hp_params)    # high-precision parameters are sharded too
    torch.manual_seed(5)
    xs = torch.randn(world * 256, 512, device=dev).bfloat16()
    ys = torch.randn(world * 256, 128 * world, device=dev).bfloat16()
    losses = []
    for _ in range(15):
        out = fsdp(xs[rank * 256:(rank + 1) * 256]) + extra.to(torch.bfloat16)
        loss = (out - ys[rank * 256:(rank + 1) * 256]).float().square().mean()
        loss.backward()
        fsdp.step(opt, clip_grad=1.0)
        losses.append(loss.item())
    torch.cuda.synchronize()
    assert native.device_status() == 0
    assert fsdp.unfused_calls == 0 and fsdp.fused_calls == 15 * 2 * 3 - 15    # every GEMM of every sharded linear (no dx for the first)
    assert losses[-1] < 0.9 * losses[0], losses
    s = fsdp.sharded[0].weight_meta.scale.clone()
    ref = s.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(s, ref)
    flat = torch.cat([p.detach().float().reshape(-1) for p in fsdp.hp_params])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(flat, ref)    # the owners' updates reached every rank
    fsdp.close()


@WORLDS
def test_full_shard_fused(world):
    _need(world)
    run_workers(_full_shard_fused, world, backend='nccl')


def _all_scenarios(rank, world):
    """Every multi-rank scenario of this file in ONE process group, one after the other (each frees its symmetric buffers
    before the next allocates its own)."""
    from msamp.nn import model_state
    scenarios = [_symm_and_barrier, _timeout_then_normal_reduce, _fp8_ddp_fused, _fused_reduce_matches_math, _zero2_training,
                 lambda r, w: _zero2_training(r, w, True, True), _fused_adam_equals_reduce_then_adam, _fused_gemms, _sp_block_fused,
                 _full_shard_fused]
    for fn in scenarios:
        fn(rank, world)
        torch.cuda.synchronize()
        dist.barrier()
        model_state.clear()


@pytest.mark.parametrize('world', [int(w) for w in os.getenv('MSAMP_TEST_COMBINED_WORLDS', '4,8').split(',') if w])
def test_all_scenarios_in_one_group(world):
    """The per-scenario tests above spawn a process group each; at four and eight ranks this test runs them all in one
    group, which costs a fraction of the GPU time and additionally covers allocate / free / re-allocate of the symmetric
    buffers in one process."""
    _need(world)
    run_workers(_all_scenarios, world, backend='nccl')
