"""LayerNorm backward through the allocation-free C entry point.

Some users of the kernel library cannot allocate device memory when they need this operator (their
memory was planned up front, or the process's allocator is not theirs to call), so
``msamp_layernorm_bwd_static`` keeps its scratch in a static device array.  The test drives the
exported C symbol directly with ctypes - no torch allocation happens between taking the pointers and
the call - and checks it against the ordinary entry point (caller-provided scratch) twice in a row,
the second time with different data, because the static scratch keeps what the previous call left.
The file name sorts last so that a run which stops at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

from msamp.ops import native

pytestmark = pytest.mark.gpu


def _run_pair(rows, cols, dtype, seed):
    lib = native.lib()
    torch.manual_seed(seed)
    dev = 'cuda'
    x = (torch.randn(rows, cols, device=dev) * 2 + 0.3).to(dtype)
    dy = torch.randn(rows, cols, device=dev).to(dtype)
    gamma = torch.rand(cols, device=dev) + 0.5
    mean = x.float().mean(1)
    rstd = torch.rsqrt(x.float().var(1, unbiased=False) + 1e-5)
    outs = []
    for static in (False, True):
        dx = torch.empty_like(x)
        dgamma = torch.empty_like(gamma)
        dbeta = torch.empty_like(gamma)
        args = [native.ptr(dy), native.ptr(x), native.ptr(gamma), native.dt(dtype), native.dt(gamma.dtype), native.ptr(mean),
                native.ptr(rstd), native.ptr(dx), native.ptr(dgamma), native.ptr(dbeta)]
        if static:
            rc = lib.msamp_layernorm_bwd_static(*args, rows, cols, native.stream())
        else:
            part = torch.empty(lib.msamp_layernorm_bwd_parts() * 2 * cols, dtype=torch.float32, device=dev)
            rc = lib.msamp_layernorm_bwd(*args, native.ptr(part), rows, cols, native.stream())
        assert rc == 0, lib.msamp_last_error().decode()
        torch.cuda.synchronize()
        outs.append((dx.float(), dgamma, dbeta))
    return outs


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
def test_static_entry_point_matches_twice(dtype):
    for seed, (rows, cols) in enumerate([(777, 4096), (130, 1024)]):    # two calls in a row share the scratch
        (dx0, dg0, db0), (dx1, dg1, db1) = _run_pair(rows, cols, dtype, seed)
        assert torch.equal(dx0, dx1)    # dx does not depend on the partial-sum layout
        scale_g = dg0.abs().max().item() + 1.0
        scale_b = db0.abs().max().item() + 1.0
        assert (dg0 - dg1).abs().max().item() <= 1e-4 * scale_g    # only the fp32 summation order differs
        assert (db0 - db1).abs().max().item() <= 1e-4 * scale_b


def test_static_entry_point_rejects_wide_rows():
    lib = native.lib()
    lib.msamp_layernorm_bwd_static.restype = ctypes.c_int
    rc = lib.msamp_layernorm_bwd_static(None, None, None, 2, 0, None, None, None, None, None, 4, 8192, None)
    assert rc == 6
    assert b'capacity' in lib.msamp_last_error()
