"""Roofline denominators measured on the box at hand: HBM copy, cuBLAS bf16, cuBLASLt FP8, NVLink peer copy, NCCL all-reduce.

    python benchmarks/bench_peaks.py                                  # one process; peer copy needs >= 2 visible GPUs
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bench_peaks.py --allreduce

Everything here is library code (``copy_``, ``torch.mm``, ``torch._scaled_mm``, ``dist.all_reduce``); the numbers are the
denominators that the fractions in the kernel benchmarks are quoted against, not results of this framework.
Timing: CUDA events on the launching stream, 3 warm-ups, 10 timed launches, buffers larger than the 126 MB L2.
"""
import argparse
import json
import os

import torch


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def single_process():
    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    n = 1 << 30
    src = torch.empty(n, dtype=torch.uint8, device=dev)
    dst = torch.empty_like(src)
    ms = timed(lambda: dst.copy_(src))
    print(json.dumps({'what': 'hbm_copy', 'bytes_moved': 2 * n, 'ms': ms, 'GBps': 2 * n / ms / 1e6}), flush=True)
    del src, dst
    shapes = {'qkv_fwd': (8192, 12288, 4096), 'proj_fwd': (8192, 4096, 4096), 'fc1_fwd': (8192, 16384, 4096), 'fc2_fwd': (8192, 4096, 16384),
              'fc1_wgrad': (16384, 4096, 8192), 'lm_head': (8192, 50304, 4096)}
    one = torch.tensor(1.0, device=dev)
    for name, (m, nn, k) in shapes.items():
        a = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
        b = torch.randn(nn, k, device=dev, dtype=torch.bfloat16)
        ms = timed(lambda: torch.mm(a, b.t()))
        print(json.dumps({'what': 'cublas_bf16', 'case': name, 'shape': [m, nn, k], 'ms': ms, 'tflops': 2.0 * m * nn * k / ms / 1e9}), flush=True)
        a8, b8 = a.to(torch.float8_e4m3fn), b.to(torch.float8_e4m3fn)
        ms = timed(lambda: torch._scaled_mm(a8, b8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16))
        print(json.dumps({'what': 'cublaslt_fp8', 'case': name, 'shape': [m, nn, k], 'ms': ms, 'tflops': 2.0 * m * nn * k / ms / 1e9}), flush=True)
        del a, b, a8, b8
    if torch.cuda.device_count() >= 2:
        n = 1 << 30
        x0 = torch.empty(n, dtype=torch.uint8, device='cuda:0')
        x1 = torch.empty(n, dtype=torch.uint8, device='cuda:1')
        ms = timed(lambda: x0.copy_(x1))    # pull over NVLink into this GPU (cudaMemcpyPeerAsync)
        print(json.dumps({'what': 'nvlink_peer_copy_one_direction', 'bytes': n, 'ms': ms, 'GBps': n / ms / 1e6}), flush=True)


def allreduce():
    import torch.distributed as dist
    rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
    torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', rank)))
    dist.init_process_group('nccl')
    for mib in (64, 256, 1024):
        x = torch.ones(mib << 18, dtype=torch.float32, device='cuda')
        dist.barrier()
        ms = timed(lambda: dist.all_reduce(x))
        t = torch.tensor([ms], device='cuda')
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            nbytes = mib << 20
            print(json.dumps({'what': 'nccl_allreduce_fp32', 'ranks': world, 'MiB': mib, 'ms': float(t), 'busbw_GBps': 2.0 * (world - 1) / world * nbytes / float(t) / 1e6}),
                  flush=True)
        del x
    dist.destroy_process_group()


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--allreduce', action='store_true')
    args = ap.parse_args()
    if args.allreduce:
        allreduce()
    else:
        single_process()
