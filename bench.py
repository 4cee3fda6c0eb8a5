"""Headline benchmark: GPT training throughput (tokens/s) with MS-AMP O2 on N B200 GPUs of one node.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Prints one JSON line (rank 0).  ``value`` is the whole-job tokens/s over K device-timed steps (CUDA
events, max over ranks) with the inputs already on the device; ``e2e`` repeats the measurement
through the public API with every step's tokens copied from pinned host memory and its loss read
back to the host.  Data are synthetic uniform token ids, weights are random-init N(0, 0.02).
``--impl reference`` runs the unmodified reference from ``baseline/_ref`` if it can be imported.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# tokens/s/GPU of the reference's published MS-AMP FP8 GPT runs (32x H100, seq 2048, micro-batch 4)
PUBLISHED_PER_GPU = {'gpt-7b': 230.5 * 2048 / 32, 'gpt-13b': 121.5 * 2048 / 32}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=6)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference', 'unfused'],
                    help="'unfused' = the reference's step sequence re-stated on library kernels (benchmarks/unfused_baseline.py): a same-box "
                         "comparison point, not the reference")
    ap.add_argument('--model', default='gpt-7b')
    ap.add_argument('--micro-batch', type=int, default=4)
    ap.add_argument('--seq', type=int, default=2048)
    ap.add_argument('--opt-level', default='O2')
    ap.add_argument('--layers', type=int, default=0, help='override the layer count (the result is then labelled as a reduced config)')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--fill-history', action='store_true',
                    help='run untimed steps until the 16-step amax histories are full, so that the timed steps use delayed scaling')
    ap.add_argument('--recompute', action='store_true', help='activation recomputation in the GPT blocks (data-parallel model only)')
    ap.add_argument('--accum', type=int, default=1, help='micro-batches per optimizer step (gradient accumulation); global batch = micro-batch x accum x DP')
    ap.add_argument('--full-shard', action='store_true', help='ZeRO-3 / FSDP full shard (default for gpt-30b on more than one GPU)')
    ap.add_argument('--overlap-comm', action='store_true', help='reduce FP8 gradients bucket by bucket during backward (data-parallel ZeRO runs)')
    ap.add_argument('--tp', type=int, default=0,
                    help='tensor-parallel size with sequence parallelism (0 = 4 for gpt-13b when the world allows it, else 1)')
    return ap.parse_args()


def reference_arm(args):
    """Run the reference through its own public API, or say in one line why that is impossible here."""
    ref = os.path.join(ROOT, 'baseline', '_ref')
    reason = None
    if not os.path.isdir(os.path.join(ref, 'msamp')):
        reason = 'baseline/_ref is empty: the reference was not installed'
    else:
        code = 'import sys; sys.path.insert(0, %r); import msamp' % ref
        res = subprocess.run([sys.executable, '-c', code], capture_output=True, text=True, cwd='/tmp')
        if res.returncode != 0:
            last = (res.stderr.strip().splitlines() or ['import failed'])[-1]
            reason = ('reference installed with --no-deps but not importable: %s (it needs deepspeed, transformer_engine v1.1 and '
                      'the MSCCL shim, none of which exist on this image or have an sm_100 build)' % last)
        else:
            reason = 'reference imports, but ships no GPT model or benchmark script to drive'
    if int(os.environ.get('RANK', '0')) == 0:
        print(json.dumps({'impl': 'reference', 'unavailable': reason}))
    return 0


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,'
              'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', '-i', str(self.index), f'--query-gpu={self.FIELDS}', '--format=csv,noheader,nounits', '-lms', '200'],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True
            )
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ''
        sm, mx, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        return {
            'sm_mhz': statistics.median(sm) if sm else None,
            'sm_max_mhz': max(mx) if mx else None,
            'samples': len(sm),
            'reasons': sorted(reasons)
        }


def main():
    args = parse()
    if args.impl == 'reference':
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    import msamp
    from msamp.models import GPT, gpt_config
    from msamp.ops import native
    from msamp.parallel import DataParallelTrainer

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        dist.init_process_group('nccl', device_id=dev)
    if world != args.gpus and rank == 0:
        print(f'warning: --gpus {args.gpus} but WORLD_SIZE={world}', file=sys.stderr)

    over = {'max_seq': args.seq}
    if args.layers:
        over['n_layer'] = args.layers
    if args.recompute:
        over['recompute'] = True
    cfg = gpt_config(args.model, **over)
    tp = args.tp or (min(4, world) if args.model == 'gpt-13b' else 1)
    full_shard = False
    dp = world // tp
    torch.manual_seed(1234)
    if args.impl == 'unfused':
        # library-kernel re-statement of the reference's step (data parallel only)
        sys.path.insert(0, os.path.join(ROOT, 'benchmarks'))
        from unfused_baseline import UnfusedGPT, UnfusedTrainer
        if tp > 1 or args.model == 'gpt-30b' or args.accum > 1:
            raise SystemExit('--impl unfused covers the data-parallel GPT configurations only')
        grp = dist.group.WORLD if world > 1 else None
        model = UnfusedGPT(cfg, dev, grp)
        trainer = UnfusedTrainer(model, lr=1e-4, betas=(0.9, 0.95), wd=0.1, group=grp)
        data_rank = rank
    elif tp > 1:
        # Megatron-style tensor + sequence parallelism inside groups of `tp` adjacent ranks, sharded optimizer over the rest
        from msamp.megatron import parallel_state as mpu
        from msamp.models import ParallelGPT
        mpu.initialize_model_parallel(tensor_model_parallel_size=tp)
        model = ParallelGPT(cfg, device=dev)    # its projections are FP8 modules already
        if args.opt_level != 'O2':
            raise SystemExit('the tensor-parallel configuration is built for --opt-level O2')
        from msamp.optim import LBAdamW
        opt = LBAdamW(model.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)    # O2: e4m3 first, fp16 second moment
        trainer = DataParallelTrainer(model, opt, zero_stage=2 if dp > 1 else 0, group=mpu.get_data_parallel_group(),
                                      after_backward=model.allreduce_sequence_parallel_grads)
        data_rank = mpu.get_data_parallel_rank()
    elif args.full_shard or (args.model == 'gpt-30b' and world > 1):
        # ZeRO-3 / FSDP full shard: FP8 weight shards, scaled-fp16 master shards and low-bit Adam states are split over
        # all ranks; the forward parameter all-gather runs inside the consuming FP8 GEMM (O3-style storage).
        from msamp.fsdp import FP8FullyShardedDataParallel
        full_shard = True
        torch.set_default_dtype(torch.bfloat16)    # the unsharded model exists only during conversion: keep it at 2 bytes
        model = GPT(cfg, device=dev)
        torch.set_default_dtype(torch.float32)
        fsdp = FP8FullyShardedDataParallel(model)
        opt = fsdp.build_optimizer(torch.optim.AdamW, lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)
        torch.cuda.empty_cache()

        class _FullShardTrainer:
            def step(self, tok, lab):
                loss = fsdp(tok, lab)
                loss.backward()
                fsdp.step(opt)
                return loss.detach()

        trainer = _FullShardTrainer()
        data_rank = rank
    else:
        model = GPT(cfg, device=dev)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)
        model, opt = msamp.initialize(model, opt, args.opt_level)
        trainer = DataParallelTrainer(model, opt, zero_stage=2 if world > 1 else 0, overlap_comm=args.overlap_comm)
        data_rank = rank

    B, S = args.micro_batch, args.seq
    gen = torch.Generator().manual_seed(data_rank)    # ranks of one tensor-parallel group see the same batch
    host_tok = [torch.randint(0, cfg.vocab_size, (B, S), generator=gen).pin_memory() for _ in range(4)]
    host_lab = [torch.randint(0, cfg.vocab_size, (B, S), generator=gen).pin_memory() for _ in range(4)]
    dev_tok = [t.to(dev) for t in host_tok]
    dev_lab = [t.to(dev) for t in host_lab]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    host_ms = [0.0]

    def timed(step_fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        calls0 = native.launch_count
        e0.record()
        h0 = time.perf_counter()
        for i in range(steps):
            step_fn(i)
        host_ms[0] = (time.perf_counter() - h0) * 1e3 / steps    # time the host needed to enqueue a step
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item(), native.launch_count - calls0

    accum = max(1, args.accum)
    if accum > 1 and not hasattr(trainer, 'step_micro_batches'):
        raise SystemExit('--accum is not available for this configuration')

    def step_device(i):
        if accum == 1:
            trainer.step(dev_tok[i % 4], dev_lab[i % 4])
        else:
            trainer.step_micro_batches([(dev_tok[(i + k) % 4], dev_lab[(i + k) % 4]) for k in range(accum)])

    last_loss = [0.0]

    def step_e2e(i):
        if accum == 1:
            tok = host_tok[i % 4].to(dev, non_blocking=True)
            lab = host_lab[i % 4].to(dev, non_blocking=True)
            loss = trainer.step(tok, lab)
        else:
            mbs = [(host_tok[(i + k) % 4].to(dev, non_blocking=True), host_lab[(i + k) % 4].to(dev, non_blocking=True)) for k in range(accum)]
            loss = trainer.step_micro_batches(mbs)
        last_loss[0] = loss.item()    # device -> host read of the step's result

    # The FP8 casts of activations and output gradients derive their scale from the tensor itself ("in-time", one
    # extra pass over the tensor) until the amax history (16 steps) is full, and from the history afterwards.  By
    # default exactly W warm-up steps run, so a short run is timed in the in-time regime; --fill-history adds untimed
    # steps first so that the timed steps are in the regime of every later step of a long run (about 2 % faster).
    fill = max(0, 17 - args.warmup) if args.fill_history else 0
    for i in range(fill):
        step_device(i)
    for i in range(args.warmup):
        step_device(i)
    sampler = ClockSampler(torch.cuda.current_device() if 'CUDA_VISIBLE_DEVICES' not in os.environ else local)
    sampler.start()
    ms, launches = timed(step_device, args.steps)
    clocks = sampler.stop()
    tokens = B * S * dp * accum * args.steps
    host_enqueue_ms = host_ms[0]
    value = tokens / (ms / 1e3)

    e2e = None
    if not args.no_e2e:
        step_e2e(0)
        ms2, _ = timed(step_e2e, args.steps)
        e2e = {
            'value': tokens / (ms2 / 1e3), 'unit': 'tokens/s', 'h2d_bytes_per_step': 2 * B * S * 8 * accum, 'd2h_bytes_per_step': 4,
            'ms_per_step': ms2 / args.steps, 'last_loss': last_loss[0]
        }
    peak_mem = torch.cuda.max_memory_allocated() / 2**30
    status = native.device_status()
    if rank == 0:
        base = PUBLISHED_PER_GPU.get(args.model)
        reduced = bool(args.layers)
        flops = cfg.flops_per_token(S) * value
        out = {
            'metric': f'tokens/sec {args.model} MS-AMP {"O3" if full_shard else args.opt_level} training' + (' (REDUCED layer count, not the headline config)' if reduced else ''),
            'value': value, 'unit': 'tokens/s', 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': ms / args.steps, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': (value / (base * world)) if (base and not reduced) else None,
            'dtype': 'fp8 GEMM (e4m3/e5m2) with bf16 activations', 'data': 'synthetic uniform token ids, random-init weights N(0,0.02)',
            'impl': 'ours' if args.impl == 'ours' else 'unfused re-statement of the reference step on library kernels (cuBLASLt FP8, ATen, SDPA, NCCL) - not the reference',
            'config': {
                'model': args.model, 'layers': cfg.n_layer, 'hidden': cfg.hidden, 'heads': cfg.n_head, 'ffn': cfg.ffn_hidden,
                'vocab': cfg.vocab_size, 'global_batch': B * dp * accum, 'micro_batch': B, 'grad_accum': accum, 'recompute': bool(args.recompute), 'seq_len': S,
                'parallelism': (f'tp{tp}+sp x ' if tp > 1 else '') + f'dp{dp}' + (('+zero3 full shard' if full_shard else '+zero2') if dp > 1 else ''),
                'opt_level': 'O3 (FP8 weight shards, fp16 master shards, FP8/fp16 Adam states)' if full_shard else args.opt_level,
                'untimed_steps_before_warmup': fill, 'scaling_regime': 'delayed (amax history full)' if fill + args.warmup >= 16 else 'in-time (first 16 steps of a run)',
                'l2': 'per-step working set (GBs of weights and activations) is far larger than the 126 MB L2, no explicit flush',
            },
            'model_tflops_per_gpu': flops / world / 1e12,
            'peak_mem_gib_per_gpu': peak_mem,
            'host_enqueue_ms_per_step': host_enqueue_ms, 'clocks': clocks, 'e2e': e2e, 'gpu_launches': launches, 'device_status': status,
        }
        if full_shard:
            # GEMMs of the sharded linears that ran the fused gather / reduce-scatter kernels vs the NCCL + plain GEMM form
            out['fused_gemm_calls'], out['unfused_gemm_calls'] = int(fsdp.fused_calls), int(fsdp.unfused_calls)
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == '__main__':
    t0 = time.time()
    sys.exit(main())
