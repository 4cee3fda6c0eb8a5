"""Helpers for multi-process tests (gloo on CPU, nccl on GPUs): spawn workers over a 127.0.0.1 rendezvous."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port():
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, backend, fn, args, errors):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['RANK'] = str(rank)
    os.environ['WORLD_SIZE'] = str(world)
    try:
        if backend == 'nccl':
            os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
            torch.cuda.set_device(rank)
            dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
        else:
            os.environ['MSAMP_DEVICE'] = 'cpu'
            dist.init_process_group('gloo', rank=rank, world_size=world)
        fn(rank, world, *args)
        dist.barrier()
    except Exception:
        errors.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_workers(fn, world=2, backend='gloo', args=()):
    """Run ``fn(rank, world, *args)`` in ``world`` processes; raise if any of them failed."""
    ctx = mp.get_context('spawn')
    errors = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, backend, fn, args, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    failed = []
    while not errors.empty():
        failed.append(errors.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            failed.append((-1, 'worker timed out'))
        elif p.exitcode != 0:
            failed.append((-1, f'worker exit code {p.exitcode}'))
    if failed:
        raise RuntimeError('\n'.join(f'[rank {r}] {msg}' for r, msg in failed))
