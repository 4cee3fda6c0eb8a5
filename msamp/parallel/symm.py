"""Symmetric memory: the same buffers allocated on every rank and mapped into every peer.

Allocation and mapping are done by the native library with CUDA IPC (``csrc/symm.cu``); the 64-byte
handles travel through ``torch.distributed`` object collectives.  Kernels receive tables of the W base
pointers and address peers directly over NVLink.
"""
import ctypes

import torch
import torch.distributed as dist

from msamp.common.utils.dist import DistUtil
from msamp.ops import native

_TYPESTR = {torch.uint8: '|u1', torch.float32: '<f4', torch.float16: '<f2', torch.int32: '<i4', torch.int64: '<i8'}


class _Exposed:
    """Minimal ``__cuda_array_interface__`` carrier so that torch can alias raw device memory."""
    def __init__(self, ptr, numel, dtype, owner):
        self.__cuda_array_interface__ = {'shape': (numel, ), 'typestr': _TYPESTR[dtype], 'data': (ptr, False), 'version': 2}
        self._owner = owner


class SymmetricBuffer:
    """``nbytes`` of zero-initialised device memory on every rank of ``group``, with peer pointers."""
    def __init__(self, nbytes, group=None):
        self.group = group
        self.world = DistUtil.get_world_size(group)
        self.rank = DistUtil.get_rank(group)
        self.nbytes = int(nbytes)
        lib = native.lib()
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        native.check(lib.msamp_symm_alloc(ctypes.c_size_t(self.nbytes), ctypes.byref(ptr), handle), 'symm_alloc')
        self.local_ptr = ptr.value
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
                self.ptrs[r] = peer.value
                self._opened.append(peer.value)
            dist.barrier(group=group)
        self.table = (ctypes.c_void_p * self.world)(*self.ptrs)
        self._device = torch.device('cuda', torch.cuda.current_device())

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
        lib = native.lib()
        for p in self._opened:
            lib.msamp_symm_close(ctypes.c_void_p(p))
        self._opened = []
        if self.local_ptr:
            lib.msamp_symm_free(ctypes.c_void_p(self.local_ptr))
            self.local_ptr = 0


class FlagPad(SymmetricBuffer):
    """Flag words for the in-kernel cross-rank barriers, plus the epoch counter every rank advances in step."""
    def __init__(self, group=None):
        super().__init__(native.lib().msamp_symm_flag_words() * 4, group)
        self.epoch = 0

    def next_epoch(self):
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
