"""Native multi-tensor low-bit Adam: builds the descriptor table and launches ``msamp_lbadam_step``."""
import ctypes

import numpy as np
import torch

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingTensor
from msamp.ops import native

_ST = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

DESC = np.dtype(
    [
        ('p', 'u8'), ('g', 'u8'), ('m', 'u8'), ('v', 'u8'),
        ('p_scale', 'u8'), ('p_scale_inv', 'u8'), ('p_amax', 'u8'),
        ('g_scale_inv', 'u8'),
        ('m_scale', 'u8'), ('m_scale_inv', 'u8'), ('m_amax', 'u8'),
        ('v_scale', 'u8'), ('v_scale_inv', 'u8'), ('v_amax', 'u8'),
        ('w8', 'u8'), ('w8_scale_inv', 'u8'),
        ('n', 'i8'),
        ('p_st', 'i4'), ('g_st', 'i4'), ('m_st', 'i4'), ('v_st', 'i4'),
        ('lr_wd_factor', 'f4'), ('l2', 'f4'), ('beta1', 'f4'), ('beta2', 'f4'), ('eps', 'f4'), ('step_size', 'f4'),
        ('inv_sqrt_bc2', 'f4'), ('gsign', 'f4'),
        ('tensor_scale', 'i4'), ('g_index', 'i4'),
        ('red', 'f4', (4, )),
    ],
    align=False
)
assert DESC.itemsize == 208


def _storage(t):
    """(value tensor, storage code, meta or None) of a Tensor / ScalingTensor."""
    if isinstance(t, ScalingTensor):
        q = t.meta.qtype
        if Dtypes.is_fp8_qtype(q):
            return t.value, (3 if q == Dtypes.kfloat8_e4m3 else 4), t.meta
        return t.value, _ST[t.value.dtype], t.meta
    return t, _ST[t.dtype], None


class FusedPlan:
    """Cached launch plan for one list of (param, state) tensors: descriptor table + block→chunk map."""
    def __init__(self, device):
        lib = native.lib()
        assert lib.msamp_lbadam_tensor_bytes() == DESC.itemsize
        self.chunk = lib.msamp_lbadam_chunk()
        self.device = device
        self.key = None
        self.ring = []    # pinned staging buffers, each with the event of the copy that last read it
        self.slot = 0
        self.dev = None
        self.work = None
        self.n_blocks = 0

    def _rebuild(self, key, sizes):
        n = len(sizes)
        # The host may run several steps ahead of the device, so the table of step k must not be
        # overwritten before its asynchronous copy has executed: rotate over a few pinned buffers
        # and wait on the event of the copy that used a buffer before refilling it.
        self.ring = []
        for _ in range(4):
            host = torch.empty(n * DESC.itemsize, dtype=torch.uint8).pin_memory()
            self.ring.append([host, host.numpy().view(DESC), None])
        self.slot = 0
        self.dev = torch.empty(n * DESC.itemsize, dtype=torch.uint8, device=self.device)
        tid, cid = [], []
        for i, sz in enumerate(sizes):
            k = max(1, (sz + self.chunk - 1) // self.chunk)
            tid.append(np.full(k, i, dtype=np.int32))
            cid.append(np.arange(k, dtype=np.int32))
        work = np.stack([np.concatenate(tid), np.concatenate(cid)], axis=1).reshape(-1)
        self.n_blocks = len(work) // 2
        self.work = torch.from_numpy(work).to(self.device)
        self.key = key

    def run(self, entries, reduce=None):
        """``entries``: list of dicts with p, g, m, v (Tensor/ScalingTensor) and the scalar hyper-parameters.

        ``reduce`` (optional): ``dict(data_table, meta_table, world, rank, n_tensors)`` of the data-parallel group's symmetric
        FP8 gradient buffers; entries with ``g_index >= 0`` then have their gradient reduce-scattered inside stage 1."""
        if not entries:
            return
        sizes = [e['p'].numel() for e in entries]
        key = tuple(sizes)
        if key != self.key:
            self._rebuild(key, sizes)
        host, a, event = self.ring[self.slot]
        if event is not None:
            event.synchronize()
        for i, e in enumerate(entries):
            pv, pst, pmeta = _storage(e['p'])
            gv, gst, gmeta = _storage(e['g'])
            mv, mst, mmeta = _storage(e['m'])
            vv, vst, vmeta = _storage(e['v'])
            if not (pv.is_contiguous() and gv.is_contiguous() and mv.is_contiguous() and vv.is_contiguous()):
                raise RuntimeError('fused Adam needs contiguous tensors')
            r = a[i]
            r['p'], r['g'], r['m'], r['v'] = pv.data_ptr(), gv.data_ptr(), mv.data_ptr(), vv.data_ptr()
            if pmeta is not None:
                r['p_scale'], r['p_scale_inv'], r['p_amax'] = pmeta.scale.data_ptr(), pmeta.scale_inv.data_ptr(), pmeta.amax.data_ptr()
            else:
                r['p_scale'] = r['p_scale_inv'] = r['p_amax'] = 0
            r['g_scale_inv'] = gmeta.scale_inv.data_ptr() if gmeta is not None else 0
            if mmeta is not None:
                r['m_scale'], r['m_scale_inv'], r['m_amax'] = mmeta.scale.data_ptr(), mmeta.scale_inv.data_ptr(), mmeta.amax.data_ptr()
            else:
                r['m_scale'] = r['m_scale_inv'] = r['m_amax'] = 0
            if vmeta is not None:
                r['v_scale'], r['v_scale_inv'], r['v_amax'] = vmeta.scale.data_ptr(), vmeta.scale_inv.data_ptr(), vmeta.amax.data_ptr()
            else:
                r['v_scale'] = r['v_scale_inv'] = r['v_amax'] = 0
            w8 = e.get('w8')
            r['w8'], r['w8_scale_inv'] = (w8[0].data_ptr(), w8[1].data_ptr()) if w8 is not None else (0, 0)
            r['n'] = sizes[i]
            r['p_st'], r['g_st'], r['m_st'], r['v_st'] = pst, gst, mst, vst
            r['lr_wd_factor'], r['l2'] = e['lr_wd_factor'], e['l2']
            r['beta1'], r['beta2'], r['eps'] = e['beta1'], e['beta2'], e['eps']
            r['step_size'], r['inv_sqrt_bc2'], r['gsign'] = e['step_size'], 1.0 / e['sqrt_bc2'], e['gsign']
            r['tensor_scale'], r['g_index'] = int(e['tensor_scale']), int(e.get('g_index', -1)) if reduce is not None else -1
            r['red'] = 0.0
        self.dev.copy_(host, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.ring[self.slot][2] = event
        self.slot = (self.slot + 1) % len(self.ring)
        if reduce is not None:
            native.check(
                native.lib().msamp_lbadam_step_reduce(
                    native.ptr(self.dev), len(entries), native.ptr(self.work), self.n_blocks, reduce['data_table'], reduce['meta_table'],
                    int(reduce['world']), int(reduce['rank']), int(reduce['n_tensors']), native.stream()
                ), 'lbadam_step_reduce'
            )
        else:
            native.check(
                native.lib().msamp_lbadam_step(native.ptr(self.dev), len(entries), native.ptr(self.work), self.n_blocks, native.stream()),
                'lbadam_step'
            )
        for e in entries:
            pv = e['p'].value if isinstance(e['p'], ScalingTensor) else e['p']
            torch.autograd.graph.increment_version(pv)


__all__ = ['FusedPlan', 'ctypes']
