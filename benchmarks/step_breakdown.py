"""Per-phase device-time breakdown of one GPT training step (O2, one GPU).

    python benchmarks/step_breakdown.py --model gpt-7b --layers 8 --warmup 3 [--delayed] [--out breakdown.json]

The step time is measured first, without any profiler, with CUDA events over three steps.  The shares come from a
second pass under ``torch.profiler`` (CUPTI kernel records of two steps): every kernel is assigned to a phase by
its name, GEMMs additionally by their position in the step (forward: qkv, proj, fc1, fc2 per layer, then lm_head;
backward: wgrad then dgrad per linear, last layer first).  Profiler durations are used as SHARES of the step only.
``--layers`` shortens the model (a 32-layer 7B step does not need to be profiled whole: the per-layer phases repeat);
the script prints both the measured short model and the extrapolation to the full layer count.
"""
import argparse
import collections
import json
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..'))
import msamp    # noqa: E402
from msamp.models import GPT, gpt_config    # noqa: E402
from msamp.parallel import DataParallelTrainer    # noqa: E402

PHASES = [
    ('gemm', ('gemm_fp8_kernel', )),
    ('attention_fwd', ('attn_fwd', )),
    ('attention_bwd', ('attn_bwd', 'attn_delta')),
    ('adam', ('lbadam', )),
    ('cast_amax', ('cast_to_fp8', 'cast_rows_colsum', 'cast_transpose', 'amax_kernel', 'transpose_bytes', 'multi_cast')),
    ('layernorm', ('layernorm', )),
    ('gelu', ('gelu_kernel', )),
    ('cross_entropy', ('xent_', )),
    ('scale_bookkeeping', ('roll_windows', 'update_scales', 'symm_', 'multi_sumsq', 'multi_clip')),
]


def phase_of(name):
    for phase, keys in PHASES:
        if any(k in name for k in keys):
            return phase
    return 'aten_other'


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='gpt-7b')
    ap.add_argument('--layers', type=int, default=8)
    ap.add_argument('--micro-batch', type=int, default=4)
    ap.add_argument('--seq', type=int, default=2048)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--delayed', action='store_true', help='warm up past the 16-step amax window so that the scales come from the history')
    ap.add_argument('--out', default=None)
    args = ap.parse_args()
    from torch.autograd import DeviceType
    from torch.profiler import ProfilerActivity, profile
    dev = torch.device('cuda', 0)
    full_layers = gpt_config(args.model).n_layer
    cfg = gpt_config(args.model, n_layer=args.layers, max_seq=args.seq)
    torch.manual_seed(0)
    model = GPT(cfg, device=dev)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4)
    model, opt = msamp.initialize(model, opt, 'O2')
    trainer = DataParallelTrainer(model, opt)
    tok = torch.randint(0, cfg.vocab_size, (args.micro_batch, args.seq), device=dev)
    for _ in range(max(args.warmup, 18 if args.delayed else 0)):
        trainer.step(tok, tok)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        trainer.step(tok, tok)
    e1.record()
    torch.cuda.synchronize()
    ms_step = e0.elapsed_time(e1) / 3
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(2):
            trainer.step(tok, tok)
        torch.cuda.synchronize()
    kern = sorted([e for e in prof.events() if e.device_type == DeviceType.CUDA and not e.name.startswith('Optimizer.step')],
                  key=lambda e: e.time_range.start)
    by_phase = collections.defaultdict(float)
    for e in kern:
        by_phase[phase_of(e.name)] += e.device_time / 2
    # GEMMs by role
    g = [e for e in kern if 'gemm_fp8_kernel' in e.name]
    g = g[:len(g) // 2]
    L = args.layers
    roles = collections.defaultdict(float)
    if len(g) == 12 * L + 3:
        for i in range(L):
            for j, nm in enumerate(('qkv', 'proj', 'fc1', 'fc2')):
                roles[f'fwd_{nm}'] += g[4 * i + j].device_time
        roles['fwd_lm_head'] = g[4 * L].device_time
        roles['wgrad_lm_head'], roles['dgrad_lm_head'] = g[4 * L + 1].device_time, g[4 * L + 2].device_time
        for i in range(L):
            for j, nm in enumerate(('wgrad_fc2', 'dgrad_fc2', 'wgrad_fc1', 'dgrad_fc1', 'wgrad_proj', 'dgrad_proj', 'wgrad_qkv', 'dgrad_qkv')):
                roles[nm] += g[4 * L + 3 + 8 * i + j].device_time
    span = (kern[-1].time_range.end - kern[0].time_range.start) / 2
    busy = sum(e.device_time for e in kern) / 2
    total = sum(by_phase.values())
    per_layer_phases = ('gemm', 'attention_fwd', 'attention_bwd', 'cast_amax', 'layernorm', 'gelu')
    fixed_gemm = roles.get('fwd_lm_head', 0) + roles.get('wgrad_lm_head', 0) + roles.get('dgrad_lm_head', 0)
    scale = ms_step * 1e3 / total    # profiler microseconds -> share of the event-timed step
    out = {'model': args.model, 'layers_measured': L, 'layers_full': full_layers, 'ms_per_step_measured_model': ms_step,
           'regime': 'delayed' if args.delayed else 'in-time', 'kernels_per_step': len(kern) / 2, 'gpu_idle_share': max(0.0, 1 - busy / span),
           'phases_ms': {k: v * scale / 1e3 for k, v in sorted(by_phase.items(), key=lambda kv: -kv[1])},
           'gemm_roles_ms': {k: v * scale / 1e3 for k, v in roles.items()}}
    if roles:
        est = 0.0
        for k, v in by_phase.items():
            v_ms = v * scale / 1e3
            if k == 'gemm':
                est += (v_ms - fixed_gemm * scale / 1e3) * full_layers / L + fixed_gemm * scale / 1e3
            elif k in per_layer_phases:
                est += v_ms * full_layers / L
            elif k == 'adam':
                n_full = gpt_config(args.model, max_seq=args.seq).num_params()
                est += v_ms * n_full / cfg.num_params()
            else:
                est += v_ms
        out['ms_per_step_extrapolated_full_model'] = est
    print(json.dumps(out, indent=1))
    if args.out:
        with open(args.out, 'w') as f:
            json.dump(out, f, indent=1)


if __name__ == '__main__':
    main()
