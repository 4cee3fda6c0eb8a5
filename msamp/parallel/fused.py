"""Fused FP8 GEMM + collective operators over symmetric memory (``csrc/gemm_fused.cu``).

``FusedGemmContext`` owns, for one process group (typically a tensor-parallel group inside one NVLink
domain): a symmetric staging buffer in which this rank exposes its shard of a sharded operand, local
buffers that receive the peers' shards, double-buffered symmetric staging for reduce-scatter, flag words
and counters.  The three operators are

* ``ag_rows_gemm``  – D = concat_r(A_r) · Bᵀ    (sequence-parallel all-gather → GEMM; with ``shard='b'``: ZeRO-3 / FSDP
  parameter all-gather → GEMM),
* ``ag_k_gemm``     – D = A · concat_r(B_r along K)ᵀ  (wgrad with a gathered, transposed activation),
* ``gemm_rs``       – reduce-scatter over ranks of the rows of A · Bᵀ (row-parallel forward, sequence-parallel dgrad).

Each has an unfused reference composition (NCCL / gloo collective + plain GEMM) used on CPU, for world
size 1, and as the oracle in the tests.
"""
import ctypes
import os

import torch
import torch.distributed as dist

from msamp.common.dtype import Dtypes
from msamp.common.utils.dist import DistUtil
from msamp.ops import gemm as _g
from msamp.ops import native

_MAXR = 8
G_NONE, G_A_ROWS, G_B_ROWS, G_B_K, G_A_K = 0, 1, 2, 3, 4


class _Desc(ctypes.Structure):
    _fields_ = [
        ('a', ctypes.c_uint64 * _MAXR), ('b', ctypes.c_uint64 * _MAXR), ('d', ctypes.c_uint64),
        ('scale_inv_a', ctypes.c_uint64), ('scale_inv_b', ctypes.c_uint64), ('bias', ctypes.c_uint64), ('amax_out', ctypes.c_uint64),
        ('M', ctypes.c_int32), ('N', ctypes.c_int32), ('K', ctypes.c_int32),
        ('a_fmt', ctypes.c_int32), ('b_fmt', ctypes.c_int32), ('out_dtype', ctypes.c_int32), ('bias_dtype', ctypes.c_int32),
        ('accumulate', ctypes.c_int32),
        ('lda', ctypes.c_int64), ('ldb', ctypes.c_int64), ('ldd', ctypes.c_int64),
        ('gather', ctypes.c_int32), ('world', ctypes.c_int32), ('rank', ctypes.c_int32), ('n_comm', ctypes.c_int32),
        ('peer', ctypes.c_uint64 * _MAXR),
        ('shard_rows', ctypes.c_int64), ('shard_pitch', ctypes.c_int64), ('shard_nrows', ctypes.c_int64),
        ('chunk_flags', ctypes.c_uint64), ('sym_flags', ctypes.c_uint64 * _MAXR),
        ('epoch', ctypes.c_uint32), ('rs', ctypes.c_int32),
        ('stage', ctypes.c_uint64 * _MAXR),
        ('rows_per_rank', ctypes.c_int32), ('pad', ctypes.c_int32),
        ('rs_out', ctypes.c_uint64), ('rs_ldo', ctypes.c_int64), ('counters', ctypes.c_uint64),
        ('limit_seconds', ctypes.c_double),
    ]


def _ptr(t):
    return 0 if t is None else t.data_ptr()


class FusedGemmContext:
    """Buffers and flags shared by the fused operators of one process group.

    Args:
        group: process group (all ranks on one NVLink domain).
        max_shard_bytes: largest operand shard that will be exposed to peers in one call (bytes).
        resident_bytes: size of the symmetric buffer that holds exposed shards (default: one shard of ``max_shard_bytes``).
            A larger buffer lets shards stay resident (e.g. the FP8 weight shards of a fully sharded model live there
            permanently, see ``resident_view``), so that no call has to copy its shard in first.
        max_out_bytes: largest full (pre-reduction) output ``M * N * itemsize`` of a ``gemm_rs`` call.
        n_comm: CTAs of the persistent grid used as copy engines in gather modes.
    """
    def __init__(self, group=None, max_shard_bytes=0, max_out_bytes=0, n_comm=12, wait_seconds=5.0, resident_bytes=0):
        self.group = group
        self.world = DistUtil.get_world_size(group)
        self.rank = DistUtil.get_rank(group)
        self.n_comm = n_comm
        self.wait_seconds = wait_seconds
        # A world of one rank runs the plain GEMM unless MSAMP_FUSED_SINGLE_RANK=1 asks for the fused kernel
        # (its copy CTAs then have nothing to fetch); that is how the kernel is profiled on one GPU.
        single_ok = os.environ.get('MSAMP_FUSED_SINGLE_RANK', '0') == '1'
        self.native = (torch.cuda.is_available() and (self.world > 1 or single_ok) and dist.is_initialized()
                       and DistUtil.backend(group) == 'nccl')
        self.max_shard_bytes = (int(max_shard_bytes) + 1023) // 1024 * 1024
        self.max_out_bytes = int(max_out_bytes)
        if not self.native:
            return
        from msamp.parallel.symm import FlagPad, SymmetricBuffer
        assert native.lib().msamp_fused_desc_bytes() == ctypes.sizeof(_Desc)
        dev = torch.device('cuda', torch.cuda.current_device())
        self.device = dev
        self.flags = FlagPad(group)
        self.resident_bytes = max(self.max_shard_bytes, (int(resident_bytes) + 1023) // 1024 * 1024)
        self.resident_used = 0
        self.shard = SymmetricBuffer(max(self.resident_bytes, 16), group) if max_shard_bytes else None
        self.local = torch.empty((self.world, max(self.max_shard_bytes, 16)), dtype=torch.uint8, device=dev) if max_shard_bytes else None
        self.stage = [SymmetricBuffer(max(self.max_out_bytes, 16), group) for _ in range(2)] if max_out_bytes else None
        self.stage_turn = 0
        self.chunk_flags = torch.zeros(self.world * 4096, dtype=torch.int32, device=dev)
        self.counters = torch.zeros(2 + self.world * 4096, dtype=torch.int32, device=dev)    # two CTA counters + one piece counter per chunk

    def reset_after_failure(self):
        """After a device-side wait gave up (``native.device_status()`` was non-zero): clear the progress counters a
        kernel may have left half-counted.  The ranks must then agree on the epoch again (``flags.epoch``) on the host."""
        if self.native:
            self.counters.zero_()

    def close(self):
        """Release the symmetric (IPC-shared) buffers.  Collective over the group, after the last fused call."""
        if not self.native:
            return
        if self.world > 1:
            dist.barrier(group=self.group)
        for buf in [self.flags, self.shard] + list(self.stage or []):
            if buf is not None:
                buf.close()
        self.flags = self.shard = self.stage = None
        self.native = False

    # ------------------------------------------------------------------ helpers
    def shard_view(self, nbytes):
        """uint8 view of this rank's exposed shard buffer (write the shard here before a gather operator)."""
        assert nbytes <= self.max_shard_bytes, (nbytes, self.max_shard_bytes)
        return self.shard.view(torch.uint8, 0, nbytes)

    def resident_view(self, nbytes):
        """Reserve ``nbytes`` of the symmetric shard buffer for good and return the uint8 view: a shard written there
        can be handed to the gather operators in every step without a copy.  Every rank must reserve in the same order."""
        off = (self.resident_used + 1023) // 1024 * 1024
        if off + nbytes > self.shard.nbytes:
            raise RuntimeError(f'resident shard buffer exhausted ({off + nbytes} > {self.shard.nbytes} bytes)')
        self.resident_used = off + nbytes
        return self.shard.view(torch.uint8, off, nbytes)

    def _shard_offset(self, t, nbytes):
        off = t.data_ptr() - self.shard.local_ptr
        assert 0 <= off and off + nbytes <= self.shard.nbytes and off % 16 == 0, \
            'the shard must live in FusedGemmContext.shard_view() / resident_view() memory'
        return off

    def _base_desc(self, M, N, K, a_q, b_q, a_sinv, b_sinv, out, bias, amax_out, accumulate):
        d = _Desc()
        d.d = _ptr(out)
        d.scale_inv_a, d.scale_inv_b = a_sinv.data_ptr(), b_sinv.data_ptr()
        d.bias = _ptr(bias)
        d.bias_dtype = 0
        d.amax_out = _ptr(amax_out)
        d.M, d.N, d.K = M, N, K
        d.a_fmt, d.b_fmt = native.fmt(a_q), native.fmt(b_q)
        d.out_dtype = native.dt(out.dtype)
        d.accumulate = int(bool(accumulate))
        d.ldd = out.stride(0) if out.dim() == 2 else N
        d.world, d.rank, d.n_comm = self.world, self.rank, self.n_comm
        d.epoch = self.flags.next_epoch()
        for r in range(self.world):
            d.sym_flags[r] = self.flags.ptrs[r]
        d.chunk_flags = self.chunk_flags.data_ptr()
        d.counters = self.counters.data_ptr()
        d.limit_seconds = self.wait_seconds
        return d

    def _launch(self, d, what):
        # A wait that gave up in an earlier kernel (a peer is late or gone) would make every later kernel of the
        # step wait for its full limit as well: stop at the first one instead.
        bits = native.peek_device_status()
        if bits:
            raise native.NativeError(f'{what}: an earlier device-side wait gave up (status bits {bits:#x}); '
                                     'read native.device_status() to clear the word after handling the failure')
        native.check(native.lib().msamp_gemm_fused(ctypes.byref(d), native.stream()), what)

    # ------------------------------------------------------------------ all-gather(rows) + GEMM
    def ag_rows_gemm(self, shard, shard_q, shard_sinv, other, other_q, other_sinv, out_dtype, bias=None, shard_is='a', out=None,
                     amax_out=None):
        """``D = gather_rows(A) · Bᵀ`` (``shard_is='a'``) or ``D = A · gather_rows(B)ᵀ`` (``shard_is='b'``).

        ``shard`` is this rank's ``[rows, K]`` FP8 block; it must already live in ``shard_view`` memory when the
        fused kernel is used (pass the view you wrote it to).  All ranks share ``shard_sinv`` (one scale).
        """
        rows, K = shard.shape
        W = self.world
        if shard_is == 'a':
            M, N = rows * W, other.shape[0]
        else:
            M, N = other.shape[0], rows * W
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=shard.device)
        tile = 128    # B row shards that are not a multiple of 256 rows make the kernel use 128 x 128 tiles
        if not self.native or rows % tile or K % 16 or rows * K > self.max_shard_bytes:
            full = all_gather_rows(shard, self.group)
            if shard_is == 'a':
                return _g.gemm_fp8(full, shard_q, shard_sinv, other, other_q, other_sinv, out_dtype, bias=bias, out=out, amax_out=amax_out)
            return _g.gemm_fp8(other, other_q, other_sinv, full, shard_q, shard_sinv, out_dtype, bias=bias, out=out, amax_out=amax_out)
        off = self._shard_offset(shard, rows * K)
        if amax_out is not None:
            amax_out.zero_()
        a_q, b_q = (shard_q, other_q) if shard_is == 'a' else (other_q, shard_q)
        a_s, b_s = (shard_sinv, other_sinv) if shard_is == 'a' else (other_sinv, shard_sinv)
        d = self._base_desc(M, N, K, a_q, b_q, a_s, b_s, out, bias, amax_out, False)
        d.gather = G_A_ROWS if shard_is == 'a' else G_B_ROWS
        nbytes = rows * K
        for r in range(W):
            ptr = self.shard.local_ptr + off if r == self.rank else self.local[r].data_ptr()
            d.peer[r] = self.shard.ptrs[r] + off
            if shard_is == 'a':
                d.a[r] = ptr
            else:
                d.b[r] = ptr
        other = other.contiguous()
        if shard_is == 'a':
            d.b[0], d.lda, d.ldb = other.data_ptr(), K, other.stride(0)
        else:
            d.a[0], d.lda, d.ldb = other.data_ptr(), other.stride(0), K
        d.shard_rows = rows
        assert nbytes <= self.max_shard_bytes
        self._launch(d, 'ag_rows_gemm')
        return out

    def gathered_rows(self, rows, K):
        """After ``ag_rows_gemm``: the full gathered operand ``[world*rows, K]`` assembled from the local copies."""
        parts = []
        for r in range(self.world):
            src = self.shard.view(torch.uint8, 0, rows * K) if r == self.rank else self.local[r][:rows * K]
            parts.append(src.view(rows, K))
        return torch.cat(parts, 0)

    # ------------------------------------------------------------------ GEMM with a K-gathered operand
    def ag_k_gemm(self, a, a_q, a_sinv, shard_t, shard_q, shard_sinv, out_dtype, out=None, accumulate=False, amax_out=None):
        """``D[M,N] = A[M, W*k] · concat_K(B_r[N, k])ᵀ`` where ``shard_t`` (``[N, k]``) is this rank's K-slice of B.

        ``shard_t`` must live in ``shard_view`` memory for the fused kernel.  Rank r's slice multiplies columns
        ``[r*k, (r+1)*k)`` of ``a``.
        """
        N, k = shard_t.shape
        W = self.world
        M, K = a.shape
        assert K == k * W
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        bn = 256 if N >= 256 else 128
        n_pad = (N + bn - 1) // bn * bn
        if not self.native or k % 128 or n_pad * k > self.max_shard_bytes:
            full = all_gather_cols(shard_t, self.group)
            return _g.gemm_fp8(a, a_q, a_sinv, full, shard_q, shard_sinv, out_dtype, out=out, accumulate=accumulate, amax_out=amax_out)
        off = self._shard_offset(shard_t, n_pad * k)
        if amax_out is not None:
            amax_out.zero_()
        a = a.contiguous()
        d = self._base_desc(M, N, K, a_q, shard_q, a_sinv, shard_sinv, out, None, amax_out, accumulate)
        d.gather = G_B_K
        for r in range(W):
            d.peer[r] = self.shard.ptrs[r] + off
            d.b[r] = self.shard.local_ptr + off if r == self.rank else self.local[r].data_ptr()
        d.a[0], d.lda, d.ldb = a.data_ptr(), a.stride(0), k
        d.shard_rows, d.shard_pitch, d.shard_nrows = k, k, N
        self._launch(d, 'ag_k_gemm')
        return out

    # ------------------------------------------------------------------ GEMM + reduce-scatter
    def gemm_rs(self, a, a_q, a_sinv, b, b_q, b_sinv, out_dtype, out=None):
        """Rows ``[rank*M/W, (rank+1)*M/W)`` of ``sum_over_ranks(A_r · B_rᵀ)``; ``a`` is ``[M, K_r]``, ``b`` is ``[N, K_r]``."""
        M, K = a.shape
        N = b.shape[0]
        W = self.world
        rows = M // W
        if out is None:
            out = torch.empty((rows, N), dtype=out_dtype, device=a.device)
        item = out.element_size()
        if not self.native or M % W or rows % 128 or (N * item) % 16 or M * N * item > self.max_out_bytes or K % 16:
            part = _g.gemm_fp8(a, a_q, a_sinv, b, b_q, b_sinv, torch.float32 if not a.is_cuda else out_dtype)
            return reduce_scatter_rows(part, self.group, out)
        a, b = a.contiguous(), b.contiguous()
        d = self._base_desc(M, N, K, a_q, b_q, a_sinv, b_sinv, out, None, None, False)
        d.a[0], d.b[0], d.lda, d.ldb = a.data_ptr(), b.data_ptr(), a.stride(0), b.stride(0)
        d.rs, d.rows_per_rank = 1, rows
        stage = self.stage[self.stage_turn]
        self.stage_turn ^= 1
        for r in range(W):
            d.stage[r] = stage.ptrs[r]
        d.rs_out, d.rs_ldo = out.data_ptr(), out.stride(0)
        self._launch(d, 'gemm_rs')
        return out


# ---------------------------------------------------------------------------------------- unfused references
def all_gather_rows(shard, group=None):
    world = DistUtil.get_world_size(group)
    if world == 1:
        return shard
    parts = [torch.empty_like(shard) for _ in range(world)]
    dist.all_gather(parts, shard.contiguous(), group=group)
    return torch.cat(parts, 0)


def all_gather_cols(shard, group=None):
    world = DistUtil.get_world_size(group)
    if world == 1:
        return shard
    parts = [torch.empty_like(shard) for _ in range(world)]
    dist.all_gather(parts, shard.contiguous(), group=group)
    return torch.cat(parts, 1)


def reduce_scatter_rows(full, group=None, out=None):
    """Sum ``full`` over ranks and keep this rank's block of rows."""
    world = DistUtil.get_world_size(group)
    rank = DistUtil.get_rank(group)
    if world == 1:
        if out is not None:
            out.copy_(full)
            return out
        return full
    rows = full.shape[0] // world
    if full.is_cuda and DistUtil.backend(group) == 'nccl':
        res = torch.empty((rows, full.shape[1]), dtype=full.dtype, device=full.device)
        dist.reduce_scatter_tensor(res, full.contiguous(), group=group)
    else:
        tmp = full.float().contiguous()
        dist.all_reduce(tmp, group=group)
        res = tmp[rank * rows:(rank + 1) * rows]
    if out is not None:
        out.copy_(res.to(out.dtype))
        return out
    return res


__all__ = ['FusedGemmContext', 'all_gather_rows', 'all_gather_cols', 'reduce_scatter_rows', 'Dtypes']
