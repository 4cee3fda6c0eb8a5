"""Symmetric memory: the same buffers allocated on every rank and mapped into every peer.

Allocation and mapping are done by the native library with CUDA IPC (``csrc/symm.cu``); the 64-byte
handles travel through ``torch.distributed`` object collectives.  Kernels receive tables of the W base
pointers and address peers directly over NVLink.
"""
import ctypes
import os

import torch
import torch.distributed as dist

from msamp.common.utils.dist import DistUtil
from msamp.ops import native

_SKEW_US = float(os.getenv('MSAMP_DEBUG_SKEW_US', '0') or 0)
_SKEW_REVERSE = os.getenv('MSAMP_DEBUG_SKEW_ORDER', '') == 'reverse'
_TYPESTR = {torch.uint8: '|u1', torch.float32: '<f4', torch.float16: '<f2', torch.int32: '<i4', torch.int64: '<i8'}


class _Exposed:
    """Minimal ``__cuda_array_interface__`` carrier so that torch can alias raw device memory."""
    def __init__(self, ptr, numel, dtype, owner):
        self.__cuda_array_interface__ = {'shape': (numel, ), 'typestr': _TYPESTR[dtype], 'data': (ptr, False), 'version': 2}
        self._owner = owner


class GuardCorruption(RuntimeError):
    """A guard region next to a symmetric buffer no longer holds its pattern: some kernel (local or a peer's) wrote
    outside the buffer."""


class SymmetricBuffer:
    """``nbytes`` of zero-initialised device memory on every rank of ``group``, with peer pointers.

    The allocation is ``GUARD`` bytes larger on either side; the two guard regions are filled with ``GUARD_BYTE`` and
    never handed to a kernel.  ``check_guards()`` (also run by ``close()``) copies them to the host and raises
    ``GuardCorruption`` when a byte changed, which is how an out-of-range peer store shows up without a memory checker.
    """
    GUARD = 4096
    GUARD_BYTE = 0xA5

    def __init__(self, nbytes, group=None):
        self.group = group
        self.world = DistUtil.get_world_size(group)
        self.rank = DistUtil.get_rank(group)
        self.nbytes = int(nbytes)
        lib = native.lib()
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        native.check(lib.msamp_symm_alloc(ctypes.c_size_t(self.nbytes + 2 * self.GUARD), ctypes.byref(ptr), handle), 'symm_alloc')
        self._base_ptr = ptr.value
        self.local_ptr = self._base_ptr + self.GUARD
        self._device = torch.device('cuda', torch.cuda.current_device())
        for g in self._guard_views():
            g.fill_(self.GUARD_BYTE)
        torch.cuda.current_stream().synchronize()    # peers may map and write the buffer right after the handle exchange
        self.ptrs = [None] * self.world
        self.ptrs[self.rank] = self.local_ptr
        self._opened = []
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                peer = ctypes.c_void_p()
                native.check(lib.msamp_symm_open(ctypes.c_char_p(h), ctypes.byref(peer)), f'symm_open(rank {r})')
                self.ptrs[r] = peer.value + self.GUARD
                self._opened.append(peer.value)
            dist.barrier(group=group)
        self.table = (ctypes.c_void_p * self.world)(*self.ptrs)

    def _guard_views(self):
        return [torch.as_tensor(_Exposed(self._base_ptr, self.GUARD, torch.uint8, self), device=self._device),
                torch.as_tensor(_Exposed(self.local_ptr + self.nbytes, self.GUARD, torch.uint8, self), device=self._device)]

    def check_guards(self):
        """Raise ``GuardCorruption`` if a byte of either guard region changed (synchronises the current stream)."""
        if not self.local_ptr:
            return
        for name, g in zip(('before', 'after'), self._guard_views()):
            bad = (g != self.GUARD_BYTE).nonzero()
            if bad.numel():
                first = int(bad[0])
                raise GuardCorruption(f'rank {self.rank}: {bad.numel()} byte(s) of the guard {name} a {self.nbytes}-byte symmetric buffer '
                                      f'were overwritten (first at guard offset {first})')

    def view(self, dtype, byte_offset=0, numel=None):
        """Tensor aliasing this rank's copy of the buffer."""
        item = torch.empty((), dtype=dtype).element_size()
        if numel is None:
            numel = (self.nbytes - byte_offset) // item
        assert byte_offset % item == 0 and byte_offset + numel * item <= self.nbytes
        if numel == 0:
            return torch.empty(0, dtype=dtype, device=self._device)
        return torch.as_tensor(_Exposed(self.local_ptr + byte_offset, numel, dtype, self), device=self._device)

    def close(self):
        """Unmap the peers' copies and free this rank's.  Collective over the group: every rank calls it, after the last
        kernel that may touch any rank's copy has completed (callers put a barrier before it).

        Freeing exported memory while a peer still has it mapped is undefined behaviour in CUDA IPC (a later allocation
        that reuses the range can lose its backing when the peer unmaps), so the ranks meet once more between "every rank
        has closed its mappings" and "every rank frees its own allocation".  A guard violation is raised only after the
        memory is released, so a rank that found one does not leave the others waiting in that barrier."""
        lib = native.lib()
        err = None
        if self.local_ptr:
            try:
                self.check_guards()
            except GuardCorruption as e:
                err = e
        for p in self._opened:
            lib.msamp_symm_close(ctypes.c_void_p(p))
        self._opened = []
        if self.local_ptr:
            if self.world > 1 and dist.is_available() and dist.is_initialized():
                dist.barrier(group=self.group)
            lib.msamp_symm_free(ctypes.c_void_p(self._base_ptr))
            self.local_ptr = 0
            self._base_ptr = 0
        if err is not None:
            raise err


class FlagPad(SymmetricBuffer):
    """Flag words for the in-kernel cross-rank barriers, plus the epoch counter every rank advances in step."""
    def __init__(self, group=None):
        super().__init__(native.lib().msamp_symm_flag_words() * 4, group)
        self.epoch = 0

    def next_epoch(self):
        """Advance the epoch; every cross-rank launch calls this right before it is enqueued.

        Debug schedules: with ``MSAMP_DEBUG_SKEW_US=<n>`` rank ``r`` first enqueues an idle spin of ``n * r`` microseconds
        (``MSAMP_DEBUG_SKEW_ORDER=reverse``: ``n * (world - 1 - r)``) on the launching stream, so the ranks reach every
        in-kernel flag exchange in a fixed, skewed order.  Two opposite orders shake out protocols that only work when
        the ranks happen to arrive together."""
        if _SKEW_US:
            k = (self.world - 1 - self.rank) if _SKEW_REVERSE else self.rank
            if k:
                torch.cuda._sleep(int(_SKEW_US * k * 1500))    # cycles; about a microsecond per 1500 at the clocks seen under load
        self.epoch += 1
        return self.epoch

    def barrier(self, slot=3, limit_seconds=10.0, announce=True):
        """Device-side barrier across the group on the current stream (bounded wait)."""
        native.check(
            native.lib().msamp_symm_barrier(
                self.table, self.rank, self.world, slot, ctypes.c_uint(self.next_epoch()), ctypes.c_double(limit_seconds), int(announce),
                native.stream()
            ), 'symm_barrier'
        )
