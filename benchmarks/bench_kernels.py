"""Single-GPU kernel benchmark: achieved throughput of each hot kernel and its fraction of the measured roofline.

    python benchmarks/bench_kernels.py [--out results.jsonl] [--profile]

``--profile`` launches every kernel once, without warm-up and on a 2 x 64 Mi-parameter optimizer case, so that the
script can be wrapped by ``ncu`` with a kernel filter (see the command lines recorded in profiles/).

Timing: CUDA events around 10 launches after 3 warm-ups; tensors are larger than the 126 MB L2 unless noted.
Denominators come from MEASURED_PEAKS.json in the repository root when present (HBM copy GB/s, cuBLAS bf16
TFLOP/s), else the fallback 6650 GB/s and 1590 TFLOP/s; FP8 GEMMs are additionally compared with cuBLASLt
(``torch._scaled_mm``) on the same shapes.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..'))
from msamp.common.dtype import Dtypes    # noqa: E402
from msamp.ops import cast, gemm    # noqa: E402
from msamp.ops import nn as K    # noqa: E402

E4, E5 = Dtypes.kfloat8_e4m3, Dtypes.kfloat8_e5m2


def peaks():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        p = json.load(open(path))
        return p['hbm_gbs'], p['bf16_tflops'], 'measured'
    return 6650.0, 1590.0, 'fallback'


PROFILE = False


def timeit(fn, iters=10, warm=3):
    if PROFILE:
        iters, warm = 1, 0
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--out', default=None)
    ap.add_argument('--profile', action='store_true')
    ap.add_argument('--only', default='', help="comma-separated subset of: gemm, stream, attention, adam")
    args = ap.parse_args()
    only = set(filter(None, args.only.split(',')))

    def want(section):
        return not only or section in only
    global PROFILE
    PROFILE = args.profile
    dev = 'cuda'
    hbm, bf16, src = peaks()
    rows = []

    def emit(**kw):
        rows.append(kw)
        print(json.dumps(kw), flush=True)

    def q(m, k, qt=E4):
        return cast.cast_to_fp8(torch.randn(m, k, device=dev), qt, torch.tensor(16.0, device=dev)), torch.tensor(1 / 16.0, device=dev)

    # ---- FP8 GEMM (GPT-7B shapes: tokens 8192).  Layouts: 'tn' = both operands K-major (forward), 'b_mn' = B stored
    # [K, N] (dgrad reads the weight as stored), 'ab_mn' = both stored [K, .] (wgrad reads dy and x as stored).
    shapes = {'qkv_fwd': (8192, 12288, 4096, 'tn'), 'proj_fwd': (8192, 4096, 4096, 'tn'), 'fc1_fwd': (8192, 16384, 4096, 'tn'),
              'fc2_fwd': (8192, 4096, 16384, 'tn'), 'fc1_dgrad': (8192, 4096, 16384, 'b_mn'), 'fc1_wgrad': (16384, 4096, 8192, 'ab_mn'),
              'lm_head': (8192, 50304, 4096, 'tn')}
    for name, (m, n, k, layout) in (shapes.items() if want('gemm') else ()):
        a_mn, b_mn = layout == 'ab_mn', layout in ('b_mn', 'ab_mn')
        a, sa = q(k, m) if a_mn else q(m, k)
        b, sb = q(k, n) if b_mn else q(n, k)
        out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        res = {}
        for label, tile in (('pair', 1), ('single', 2)):
            res[label] = timeit(lambda: gemm.gemm_fp8(a, E4, sa, b, E4, sb, torch.bfloat16, out=out, a_mn=a_mn, b_mn=b_mn, tile=tile))
        ms = timeit(lambda: gemm.gemm_fp8(a, E4, sa, b, E4, sb, torch.bfloat16, out=out, a_mn=a_mn, b_mn=b_mn))
        a8 = (a.t() if a_mn else a).view(torch.float8_e4m3fn)
        b8 = (b if b_mn else b.t()).view(torch.float8_e4m3fn)
        try:
            # cuBLASLt wants A row-major and B column-major: give it materialised copies in that layout
            a8c = a8.contiguous()
            b8c = b8.t().contiguous().t()
            ms_ref = None if PROFILE else timeit(lambda: torch._scaled_mm(a8c, b8c, scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16))
        except Exception:
            ms_ref = None
        tf = 2 * m * n * k / ms / 1e9
        emit(kernel='gemm_fp8', case=name, layout=layout, shape=[m, n, k], ms=ms, ms_pair=res['pair'], ms_single=res['single'], tflops=tf,
             frac_of_bf16_peak=tf / bf16, peak_source=src, cublaslt_ms=ms_ref, vs_cublaslt=(ms_ref / ms) if ms_ref else None)

    # ---- bandwidth-bound kernels on [8192*4, 4096] bf16 (256 MB)
    if want('stream'):
        x = torch.randn(32768, 4096, device=dev, dtype=torch.bfloat16)
        s = torch.tensor(8.0, device=dev)
        am = torch.zeros((), device=dev)
        n = x.numel()
        cases = {
            'amax': (lambda: cast.amax(x, am), 2 * n),
            'cast_to_fp8': (lambda: cast.cast_to_fp8(x, E4, s, am), 3 * n),
            'cast_transpose_fp8': (lambda: cast.cast_transpose_fp8(x, E4, s, am), 4 * n),
            'cast_transpose_fp8_t_only': (lambda: cast.cast_transpose_fp8(x, E5, s, am, need_rowmajor=False), 3 * n),
        }
        x8 = cast.cast_to_fp8(x, E4, s)
        cases['transpose_fp8'] = (lambda: cast.transpose_fp8(x8), 2 * n)
        cases['cast_from_fp8'] = (lambda: cast.cast_from_fp8(x8, E4, s, torch.bfloat16), 3 * n)
        w = torch.ones(4096, device=dev)
        bb = torch.zeros(4096, device=dev)
        cases['layernorm_fwd'] = (lambda: K.layer_norm(x, w, bb), 4 * n)
        cases['gelu_fwd'] = (lambda: K.gelu(x), 4 * n)
        for name, (fn, nbytes) in cases.items():
            with torch.no_grad():
                ms = timeit(fn)
            gbs = nbytes / ms / 1e6
            emit(kernel=name, bytes=nbytes, ms=ms, gbs=gbs, frac_of_hbm_copy=gbs / hbm, peak_source=src)
        xg = x.clone().requires_grad_()
        y = K.layer_norm(xg, w.requires_grad_(), bb.requires_grad_())
        dy = torch.randn_like(y)
        ms = timeit(lambda: torch.autograd.grad(y, xg, dy, retain_graph=True))
        emit(kernel='layernorm_bwd', bytes=6 * n, ms=ms, gbs=6 * n / ms / 1e6, frac_of_hbm_copy=6 * n / ms / 1e6 / hbm, peak_source=src)

    # ---- attention (GPT-7B layer: batch 4, seq 2048, 32 heads of 128), causal
    if want('attention'):
        qkv = torch.randn(4, 2048, 3, 32, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
        with torch.no_grad():
            ms_f = timeit(lambda: K.attention_qkv(qkv, causal=True))
        o = K.attention_qkv(qkv, causal=True)
        do = torch.randn_like(o)
        ms_b = timeit(lambda: torch.autograd.grad(o, qkv, do, retain_graph=True))
        fl_f = 4 * 4 * 32 * 2048 * 2048 * 128 / 2
        emit(kernel='attention_fwd', ms=ms_f, tflops=fl_f / ms_f / 1e9, frac_of_bf16_peak=fl_f / ms_f / 1e9 / bf16, peak_source=src)
        emit(kernel='attention_bwd', ms=ms_b, tflops=2.5 * fl_f / ms_b / 1e9, frac_of_bf16_peak=2.5 * fl_f / ms_b / 1e9 / bf16, peak_source=src,
             note='useful FLOPs (5 GEMMs); the two-kernel backward recomputes the scores twice')

    # ---- fused LBAdam over 1 Gi parameters (O2 layout: fp16 scaled weight, e4m3 grad, e4m3 m, fp16 v)
    if want('adam'):
        from msamp.nn import ScalingParameter
        from msamp.optim import LBAdamW
        ps = [ScalingParameter((torch.randn(16384, 8192 if not PROFILE else 4096, device=dev) * 0.02).cast(Dtypes.kfloat16))
              for _ in range(8 if not PROFILE else 2)]
        opt = LBAdamW(ps, lr=1e-4)
        for p in ps:
            p.grad = (torch.randn(*p.shape, device=dev) * 1e-3).cast(E4)
        opt.step()
        ms = timeit(lambda: opt.lb_step(), iters=5, warm=2)
        npar = sum(p.numel() for p in ps)
        nbytes = npar * (6 + 6 + 5)
        emit(kernel='lbadam_step', params=npar, ms=ms, gbs=nbytes / ms / 1e6, frac_of_hbm_copy=nbytes / ms / 1e6 / hbm, peak_source=src,
             note='two passes: 6+6 bytes read, 5 bytes written per parameter')
    if args.out:
        with open(args.out, 'w') as f:
            for r in rows:
                f.write(json.dumps(r) + '\n')


if __name__ == '__main__':
    main()
