"""FP8 gradient all-reduce / reduce-scatter sweep (1 MB - 1 GB of bf16 gradients) on N GPUs of one node.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node N benchmarks/bench_grad_reduce.py

Buckets hold values ~N(0, 1e-3) with 0.1 % outliers scaled x100.  Two implementations are timed on the device
(CUDA events, max over ranks, 3 warm-ups):

* ``fused``     msamp_symm_grad_reduce: one kernel that waits for the peers, pulls their e4m3 bytes over NVLink, dequantises
                with each peer's scale, averages in fp32, re-quantises once (reduce-scatter) and optionally writes the
                result to every peer (all-reduce).  The e4m3 quantisation of the local bucket is timed with it.
* ``reference`` the reference's sequence with stock collectives: amax MAX all-reduce, quantise with the common scale, NCCL
                sum of the FP8 numbers (all_reduce / reduce_scatter on float8_e4m3fn), divide scale_inv.

Bus bandwidth uses the NCCL convention on the FP8 payload: all-reduce 2(N-1)/N * bytes / t, reduce-scatter (N-1)/N * bytes / t.
Roofline: bytes that must cross NVLink per GPU divided by 770 GB/s (measured peer-copy bandwidth on this machine).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..'))
from msamp.common.dtype import Dtypes    # noqa: E402
from msamp.ops import cast, native    # noqa: E402
from msamp.parallel.symm import FlagPad, SymmetricBuffer    # noqa: E402

E4 = Dtypes.kfloat8_e4m3
LINK_GBS = 770.0


def main():
    import ctypes
    ap = argparse.ArgumentParser()
    ap.add_argument('--max-mb', type=int, default=1024)
    ap.add_argument('--out', default=None)
    args = ap.parse_args()
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    dist.init_process_group('nccl', device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    lib = native.lib()
    chunk = lib.msamp_symm_chunk_bytes()
    sizes_mb = [s for s in (1, 4, 16, 64, 256, 1024) if s <= args.max_mb]
    max_elems = sizes_mb[-1] * (1 << 20) // 2
    g_buf = SymmetricBuffer(max_elems)
    g_meta = SymmetricBuffer(3 * 8 * 4)
    flags = FlagPad()
    results = []

    def timed(fn, iters=10, warm=3):
        for _ in range(warm):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    for mb in sizes_mb:
        n = mb * (1 << 20) // 2    # bf16 elements == e4m3 bytes
        gen = torch.Generator(device=dev).manual_seed(1000 + rank)
        grad = torch.randn(n, device=dev, generator=gen) * 1e-3
        outl = torch.rand(n, device=dev, generator=gen) < 1e-3
        grad = torch.where(outl, grad * 100, grad).bfloat16()
        flat = g_buf.view(torch.uint8, 0, n)
        meta = g_meta.view(torch.float32).view(3, 8)
        scale = torch.ones((), device=dev)
        # one logical tensor; every rank owns an equal share of its chunks
        n_chunks = (n + chunk - 1) // chunk
        mine = [c for c in range(n_chunks) if c * world // n_chunks == rank] if n_chunks >= world else ([0] if rank == 0 else [])
        work_rs = torch.tensor([(0, c) for c in mine] or [(0, 0)], dtype=torch.int32, device=dev).reshape(-1)
        n_work = len(mine)
        offsets = torch.tensor([0, (n + 15) // 16 * 16], dtype=torch.int64, device=dev)

        def fused(broadcast):
            cast.amax_and_scale(grad, meta[1, 0:1].view(()), scale, meta[0, 0:1].view(()), E4)
            cast.cast_to_fp8(grad, E4, scale, out=flat)
            native.check(lib.msamp_symm_grad_reduce(g_buf.table, g_meta.table, flags.table, native.ptr(offsets), native.ptr(work_rs), n_work,
                                                    8, rank, world, ctypes.c_uint(flags.next_epoch()), broadcast, ctypes.c_double(30.0), 0,
                                                    native.stream()), 'grad_reduce')

        ref_buf = torch.empty(n, dtype=torch.uint8, device=dev)
        ref_out = torch.empty(n // world, dtype=torch.uint8, device=dev)
        amax = torch.zeros((), device=dev)
        rscale, rsinv = torch.ones((), device=dev), torch.ones((), device=dev)

        def reference(broadcast):
            cast.amax(grad, amax)
            dist.all_reduce(amax, op=dist.ReduceOp.MAX)
            cast.update_scales(amax.view(1), rscale.view(1), rsinv.view(1), E4)
            rscale.mul_(1.0 / world**0.5)
            cast.cast_to_fp8(grad, E4, rscale, out=ref_buf)
            if broadcast:
                dist.all_reduce(ref_buf.view(torch.float8_e4m3fn))
            else:
                dist.reduce_scatter_tensor(ref_out.view(torch.float8_e4m3fn), ref_buf[:ref_out.numel() * world].view(torch.float8_e4m3fn))
            rsinv.div_(world)

        for op, broadcast in (('all_reduce', 1), ('reduce_scatter', 0)):
            t_f = timed(lambda: fused(broadcast))
            try:
                t_r = timed(lambda: reference(broadcast))
            except Exception as e:    # NCCL build without float8 reductions
                t_r, err = None, repr(e)[:80]
            factor = (2 * (world - 1) / world) if broadcast else ((world - 1) / world)
            bus = factor * n / t_f / 1e6
            link_bytes = n * (world - 1) / world * (2 if broadcast else 1)    # per GPU, per direction the heavier of in/out
            roof_ms = link_bytes / LINK_GBS / 1e6
            rec = {'op': op, 'gpus': world, 'bf16_mb': mb, 'fp8_bytes': n, 'fused_ms': t_f, 'fused_bus_gbs': bus, 'reference_ms': t_r,
                   'reference_bus_gbs': (factor * n / t_r / 1e6) if t_r else None, 'speedup': (t_r / t_f) if t_r else None,
                   'roofline_ms': roof_ms, 'roofline_frac': roof_ms / t_f}
            results.append(rec)
            if rank == 0:
                print(json.dumps(rec), flush=True)
        torch.cuda.synchronize()
        assert native.device_status() == 0
    if rank == 0 and args.out:
        with open(args.out, 'w') as f:
            for r in results:
                f.write(json.dumps(r) + '\n')
    dist.barrier()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
