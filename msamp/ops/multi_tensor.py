"""Multi-tensor gradient norm, overflow flag and clipping over mixed high-precision / FP8 gradients.

``grad_sumsq(grads)`` and ``clip_by_sumsq(grads, sumsq, max_norm)`` each cost one kernel launch for any number of
tensors on CUDA (``csrc/multi_tensor.cu``); CPU tensors take the same arithmetic in plain torch.  A gradient is a
``torch.Tensor`` (fp32 / fp16 / bf16) or a ``ScalingTensor`` whose payload is e4m3 / e5m2 (clipped through its
``scale_inv``) or a scaled 16-bit tensor (handled like a plain tensor times ``scale_inv``).
"""
import numpy as np
import torch

from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingTensor
from msamp.ops import native

_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
_DESC = np.dtype([('data', 'u8'), ('scale_inv', 'u8'), ('n', 'i8'), ('code', 'i4'), ('pad', 'i4')], align=False)
_CAST_DESC = np.dtype([('src', 'u8'), ('dst', 'u8'), ('scale', 'u8'), ('scale_inv', 'u8'), ('amax_in', 'u8'), ('amax_out', 'u8'), ('n', 'i8'),
                       ('code', 'i4'), ('fmt', 'i4')], align=False)


class _Table:
    """Descriptor table + work list in device memory, refilled through a ring of pinned host buffers so that the host
    may run ahead of the device without overwriting a table an earlier launch still has to read."""
    def __init__(self, device, desc=None, size_field=2):
        self.device = device
        self.desc = desc if desc is not None else _DESC
        self.size_field = size_field    # position of the element count in a row tuple
        self.cap = 0
        self.ring = []
        self.slot = 0
        self.work_key = None
        self.work = None
        self.n_work = 0

    def fill(self, rows):
        n = len(rows)
        if n > self.cap:
            self.cap = max(64, 2 * n)
            self.ring = []
            for _ in range(4):
                host = torch.empty(self.cap * self.desc.itemsize, dtype=torch.uint8).pin_memory()
                self.ring.append([host, host.numpy().view(self.desc), None,
                                  torch.empty(self.cap * self.desc.itemsize, dtype=torch.uint8, device=self.device)])
            self.slot = 0
        host, arr, event, dev = self.ring[self.slot]
        if event is not None:
            event.synchronize()
        names = self.desc.names
        for i, row in enumerate(rows):
            r = arr[i]
            for name, v in zip(names, row):
                r[name] = v
        dev[:n * self.desc.itemsize].copy_(host[:n * self.desc.itemsize], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.ring[self.slot][2] = ev
        self.slot = (self.slot + 1) % len(self.ring)
        key = tuple(r[self.size_field] for r in rows)
        if key != self.work_key:
            chunk = native.lib().msamp_multi_tensor_chunk()
            tid, cid = [], []
            for i, r in enumerate(rows):
                k = max(1, (r[self.size_field] + chunk - 1) // chunk)
                tid.append(np.full(k, i, dtype=np.int32))
                cid.append(np.arange(k, dtype=np.int32))
            work = np.stack([np.concatenate(tid), np.concatenate(cid)], axis=1).reshape(-1)
            self.n_work = len(work) // 2
            self.work = torch.from_numpy(work).to(self.device)
            self.work_key = key
        return dev


_tables = {}


def _rows(grads):
    rows = []
    for g in grads:
        if isinstance(g, ScalingTensor):
            v = g.value
            if not v.is_contiguous():
                raise RuntimeError('multi-tensor kernels need contiguous gradients')
            if Dtypes.is_fp8_qtype(g.qtype):
                code = 3 if g.qtype == Dtypes.kfloat8_e4m3 else 4
            else:
                code = _CODE[v.dtype]
            rows.append((v.data_ptr(), g.meta.scale_inv.data_ptr(), v.numel(), code, 0))
        else:
            if not g.is_contiguous():
                raise RuntimeError('multi-tensor kernels need contiguous gradients')
            rows.append((g.data_ptr(), 0, g.numel(), _CODE[g.dtype], 0))
    return rows


def _table_for(grads, tag):
    dev = (grads[0].value if isinstance(grads[0], ScalingTensor) else grads[0]).device
    key = (dev, tag)
    t = _tables.get(key)
    if t is None:
        t = _tables[key] = _Table(dev)
    return t, dev


def grad_sumsq(grads, out=None, tag='default'):
    """``out[0] += sum over all gradients of |dequantised value|^2``; ``out[1] = 1`` if any value is inf / NaN.

    ``out`` is a 2-element fp32 tensor (created zeroed when omitted).  ``tag`` keeps separate cached tables for call
    sites that alternate between different tensor lists.
    """
    grads = [g for g in grads if g is not None]
    first = (grads[0].value if isinstance(grads[0], ScalingTensor) else grads[0]) if grads else None
    if out is None:
        out = torch.zeros(2, dtype=torch.float32, device=first.device if first is not None else 'cpu')
    if not grads:
        return out
    if first.is_cuda:
        table, _ = _table_for(grads, tag)
        dev_rows = table.fill(_rows(grads))
        native.check(
            native.lib().msamp_multi_tensor_sumsq(native.ptr(dev_rows), native.ptr(table.work), table.n_work, native.ptr(out), native.stream()),
            'multi_tensor_sumsq'
        )
        return out
    for g in grads:
        if isinstance(g, ScalingTensor):
            if Dtypes.is_fp8_qtype(g.qtype):
                v = g.value.view(torch.uint8).view(Dtypes.qtype_to_float8[g.qtype]).float()
            else:
                v = g.value.float()
            s = v.square().sum() * g.meta.scale_inv.float().square()
        else:
            s = g.detach().float().square().sum()
        out[0] += s
        if not bool(torch.isfinite(s)):
            out[1] = 1.0
    return out


def clip_by_sumsq(grads, sumsq, max_norm, eps=1e-6, tag='default'):
    """Multiply every gradient by ``min(1, max_norm / (sqrt(sumsq) + eps))``; FP8 gradients only change ``scale_inv``.

    ``sumsq`` is a 0-d / 1-element fp32 tensor on the gradients' device (typically ``grad_sumsq(...)[0:1]`` after the
    cross-rank reductions)."""
    grads = [g for g in grads if g is not None]
    if not grads:
        return
    first = grads[0].value if isinstance(grads[0], ScalingTensor) else grads[0]
    if first.is_cuda:
        table, _ = _table_for(grads, tag)
        dev_rows = table.fill(_rows(grads))
        native.check(
            native.lib().msamp_multi_tensor_clip(
                native.ptr(dev_rows), native.ptr(table.work), table.n_work, native.ptr(sumsq), native.ctypes_float(max_norm),
                native.ctypes_float(eps), native.stream()
            ), 'multi_tensor_clip'
        )
        return
    coef = torch.clamp(max_norm / (sumsq.reshape(()).sqrt() + eps), max=1.0)
    if float(coef) >= 1.0:
        return
    for g in grads:
        if isinstance(g, ScalingTensor):
            g.meta.scale_inv.mul_(coef)
        else:
            g.detach().mul_(coef.to(g.dtype))


def cast_to_fp8_multi(srcs, dsts, qtype, scales, scale_invs=None, amax_ins=None, amax_outs=None, tag='cast'):
    """Quantise several high-precision tensors to FP8 in ONE launch, each with its own scale.

    ``srcs[i]`` (fp32 / fp16 / bf16, contiguous) → ``dsts[i]`` (uint8, same number of elements) with ``scales[i]``.
    With ``amax_ins[i]`` the scale is first derived from that amax by the power-of-two rule and stored (in-time scaling from
    an amax the producer reduced); ``amax_outs[i]`` receives ``max|src|`` (delayed scaling); ``scale_invs[i]`` receives
    ``1 / scale``.  All scalars are 0-d fp32 tensors on the tensors' device.
    """
    n = len(srcs)
    if n == 0:
        return
    pick = lambda seq, i: (seq[i] if seq is not None else None)    # noqa: E731
    if srcs[0].is_cuda:
        assert native.lib().msamp_multi_tensor_cast_desc_bytes() == _CAST_DESC.itemsize
        dev = srcs[0].device
        key = (dev, 'cast:' + tag)
        table = _tables.get(key)
        if table is None:
            table = _tables[key] = _Table(dev, _CAST_DESC, size_field=6)
        rows = []
        fmt = native.fmt(qtype)
        for i in range(n):
            src, dst = srcs[i], dsts[i]
            if not (src.is_contiguous() and dst.is_contiguous()) or dst.numel() != src.numel() or dst.dtype != torch.uint8:
                raise RuntimeError('cast_to_fp8_multi needs contiguous tensors and uint8 destinations of the same size')
            ptr = lambda t: (t.data_ptr() if t is not None else 0)    # noqa: E731
            if amax_outs is not None and amax_outs[i] is not None:
                amax_outs[i].zero_()
            rows.append((src.data_ptr(), dst.data_ptr(), scales[i].data_ptr(), ptr(pick(scale_invs, i)), ptr(pick(amax_ins, i)),
                         ptr(pick(amax_outs, i)), src.numel(), _CODE[src.dtype], fmt))
        dev_rows = table.fill(rows)
        native.check(native.lib().msamp_multi_tensor_cast(native.ptr(dev_rows), native.ptr(table.work), table.n_work, native.stream()),
                     'multi_tensor_cast')
        return
    from msamp.ops import cast as _c
    for i in range(n):
        _c.cast_to_fp8(srcs[i], qtype, scales[i], pick(amax_outs, i), scale_inv_out=pick(scale_invs, i), amax_in=pick(amax_ins, i),
                       out=dsts[i].view(-1))
