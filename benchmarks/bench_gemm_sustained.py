"""Sustained FP8 GEMM throughput under the power cap, with the SM clock seen while it ran.

    python benchmarks/bench_gemm_sustained.py [--iters 3000] [--shape 8192,12288,4096]

A burst of a few launches runs at boost clocks; inside a training step the GEMMs run back to back for hundreds of
milliseconds and the 1 kW power limit pulls the SM clock down.  This script runs each variant (our kernel with the
single-CTA 128x256 tile, with the CTA-pair 256x256 tile, and cuBLASLt FP8 through ``torch._scaled_mm``) for thousands
of launches, samples ``nvidia-smi`` every 100 ms meanwhile (read-only) and prints the achieved TFLOP/s, the median SM
clock under load and TFLOP/s per GHz, which separates "does more work per clock" from "is allowed a higher clock".
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..'))
from msamp.common.dtype import Dtypes    # noqa: E402
from msamp.ops import cast, gemm    # noqa: E402

QUERY = 'clocks.sm,power.draw,clocks_event_reasons.sw_power_cap'


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--iters', type=int, default=3000)
    ap.add_argument('--shape', default='8192,12288,4096', help='M,N,K of D[M,N] = A[M,K] B[N,K]^T')
    args = ap.parse_args()
    m, n, k = (int(v) for v in args.shape.split(','))
    dev = torch.device('cuda', 0)
    e4 = Dtypes.kfloat8_e4m3

    def quantised(rows, cols):
        return cast.cast_to_fp8(torch.randn(rows, cols, device=dev), e4, torch.tensor(16.0, device=dev)), torch.tensor(1 / 16.0, device=dev)

    a, sa = quantised(m, k)
    b, sb = quantised(n, k)
    out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
    a8, b8 = a.view(torch.float8_e4m3fn), b.view(torch.float8_e4m3fn)
    variants = {
        'ours_single_cta_128x256': lambda: gemm.gemm_fp8(a, e4, sa, b, e4, sb, torch.bfloat16, out=out, tile=2),
        'ours_cta_pair_256x256': lambda: gemm.gemm_fp8(a, e4, sa, b, e4, sb, torch.bfloat16, out=out, tile=1),
        'cublaslt_fp8': lambda: torch._scaled_mm(a8, b8.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16),
    }
    for name, fn in variants.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        smi = subprocess.Popen(['nvidia-smi', '-i', '0', f'--query-gpu={QUERY}', '--format=csv,noheader,nounits', '-lms', '100'],
                               stdout=subprocess.PIPE, text=True)
        time.sleep(0.3)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.iters
        smi.terminate()
        text, _ = smi.communicate()
        rows = [line.split(',') for line in text.strip().splitlines()]
        rows = [r for r in rows if len(r) >= 3]
        loaded = [(float(r[0]), float(r[1]), r[2].strip()) for r in rows if float(r[1]) > 500.0]
        tflops = 2.0 * m * n * k / ms / 1e9
        rec = {'variant': name, 'shape': [m, n, k], 'ms': ms, 'tflops': tflops, 'samples_under_load': len(loaded)}
        if loaded:
            clk = statistics.median(c for c, _, _ in loaded)
            rec.update(sm_mhz_median=clk, power_w_max=max(p for _, p, _ in loaded), tflops_per_ghz=tflops / (clk / 1000.0),
                       sw_power_cap_active=any(r == 'Active' for _, _, r in loaded))
        print(json.dumps(rec), flush=True)
        time.sleep(2)    # let the package cool to the same starting point for the next variant


if __name__ == '__main__':
    main()
