"""Fused GEMM + collective kernels against the unfused composition (NCCL collective, then GEMM) on one node.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node N benchmarks/bench_fused_gemm.py [--hidden 5120 --ffn 20480 --tokens 8192]

Shapes are those of a GPT block under tensor + sequence parallelism over the N ranks (defaults: GPT-13B, 8192 tokens).
For each path: device time of the fused kernel, of the unfused pair, and the roofline - the slower of
(FLOPs / measured FP8 GEMM rate of the plain kernel on the same shape) and (bytes over NVLink per GPU / 770 GB/s).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..'))
from msamp.common.dtype import Dtypes    # noqa: E402
from msamp.ops import cast, gemm, native    # noqa: E402
from msamp.parallel.fused import FusedGemmContext, all_gather_cols, all_gather_rows, reduce_scatter_rows    # noqa: E402

E4, E5 = Dtypes.kfloat8_e4m3, Dtypes.kfloat8_e5m2
LINK_GBS = 770.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--hidden', type=int, default=5120)
    ap.add_argument('--ffn', type=int, default=20480)
    ap.add_argument('--tokens', type=int, default=8192)
    ap.add_argument('--n-comm', type=int, default=12)
    ap.add_argument('--out', default=None)
    args = ap.parse_args()
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    dist.init_process_group('nccl', device_id=dev)
    rank, W = dist.get_rank(), dist.get_world_size()
    H, F, T = args.hidden, args.ffn, args.tokens
    m = T // W
    ctx = FusedGemmContext(None, max_shard_bytes=max(m * F, (F // W + 256) * m, (H + 256) * m), max_out_bytes=T * max(H, F // W) * 2,
                           n_comm=args.n_comm)
    sinv = torch.tensor(1 / 16.0, device=dev)
    s16 = torch.tensor(16.0, device=dev)
    results = []

    def q(shape, seed, qt=E4):
        g = torch.Generator(device=dev).manual_seed(seed)
        return cast.cast_to_fp8(torch.randn(*shape, device=dev, generator=g), qt, s16)

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

    def report(name, fused, unfused, plain, flops, link_bytes):
        t_f, t_u, t_p = timed(fused), timed(unfused), timed(plain)
        roof = max(t_p, link_bytes / LINK_GBS / 1e6)
        rec = {'path': name, 'gpus': W, 'fused_ms': t_f, 'unfused_ms': t_u, 'plain_gemm_ms': t_p, 'speedup_vs_unfused': t_u / t_f,
               'tflops_fused': flops / t_f / 1e9, 'nvlink_bytes_per_gpu': link_bytes, 'roofline_ms': roof, 'roofline_frac': roof / t_f}
        results.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)

    # ---- column-parallel forward: y[T, F/W] = all-gather-rows(x8[m, H]) . W[F/W, H]^T
    x8 = q((m, H), 1 + rank)
    w_col = q((F // W, H), 50)
    view = ctx.shard_view(m * H).view(m, H)
    view.copy_(x8)
    full_x = all_gather_rows(x8)
    report('ag_rows_gemm (SP forward, X18+GEMM)',
           lambda: ctx.ag_rows_gemm(view, E4, sinv, w_col, E4, sinv, torch.bfloat16),
           lambda: gemm.gemm_fp8(all_gather_rows(x8), E4, sinv, w_col, E4, sinv, torch.bfloat16),
           lambda: gemm.gemm_fp8(full_x, E4, sinv, w_col, E4, sinv, torch.bfloat16),
           2 * T * (F // W) * H, m * H * (W - 1))
    # ---- column-parallel dgrad: dx[m, H] = reduce-scatter-rows(dy8[T, F/W] . W^T[H, F/W]^T)
    dy8 = q((T, F // W), 3, E5)
    w_col_t = q((H, F // W), 51)
    report('gemm_rs (SP dgrad, GEMM+X21)',
           lambda: ctx.gemm_rs(dy8, E5, sinv, w_col_t, E4, sinv, torch.bfloat16),
           lambda: reduce_scatter_rows(gemm.gemm_fp8(dy8, E5, sinv, w_col_t, E4, sinv, torch.bfloat16)),
           lambda: gemm.gemm_fp8(dy8, E5, sinv, w_col_t, E4, sinv, torch.bfloat16),
           2 * T * H * (F // W), m * H * 2 * (W - 1))
    # ---- column-parallel wgrad: dW[F/W, H] = dy8^T[F/W, T] . all-gather-K(x8^T[H, m])^T
    dy8t = q((F // W, T), 4, E5)
    x8t = q((H, m), 5 + rank)
    rows_pad = (H + 255) // 256 * 256
    view_t = ctx.shard_view(rows_pad * m)[:H * m].view(H, m)
    view_t.copy_(x8t)
    full_xt = all_gather_cols(x8t)
    report('ag_k_gemm (SP wgrad, X19+GEMM)',
           lambda: ctx.ag_k_gemm(dy8t, E5, sinv, view_t, E4, sinv, torch.bfloat16),
           lambda: gemm.gemm_fp8(dy8t, E5, sinv, all_gather_cols(x8t), E4, sinv, torch.bfloat16),
           lambda: gemm.gemm_fp8(dy8t, E5, sinv, full_xt, E4, sinv, torch.bfloat16),
           2 * (F // W) * H * T, m * H * (W - 1))
    # ---- ZeRO-3 / FSDP forward: y[T, F] = x8[T, H] . all-gather-rows(W_r[F/W, H])^T
    xa = q((T, H), 7)
    w_shard = q((F // W, H), 60 + rank)
    view_w = ctx.shard_view((F // W) * H).view(F // W, H)
    view_w.copy_(w_shard)
    full_w = all_gather_rows(w_shard)
    report('param ag_rows_gemm (ZeRO-3 forward, X10+GEMM)',
           lambda: ctx.ag_rows_gemm(view_w, E4, sinv, xa, E4, sinv, torch.bfloat16, shard_is='b'),
           lambda: gemm.gemm_fp8(xa, E4, sinv, all_gather_rows(w_shard), E4, sinv, torch.bfloat16),
           lambda: gemm.gemm_fp8(xa, E4, sinv, full_w, E4, sinv, torch.bfloat16),
           2 * T * F * H, (F // W) * H * (W - 1))
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
