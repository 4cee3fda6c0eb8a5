"""Process-wide registry of the scaling metas of all FP8 linears.

The metas of one kind (``input`` / ``wgrad`` / ``ograd``) are laid out in contiguous buffers
``scales[n]``, ``scales_inv[n]``, ``amaxs[n, window]``, ``amax_counters[n]`` so that the delayed-scaling
update of every layer is one kernel launch.  Each ScalingMeta keeps views into those buffers and
is ``locked``: replacing its tensors would silently detach it from the flat storage, so
``check_metas_in_flat`` verifies the aliasing by address.  (reference: msamp/nn/state.py:12-194)
"""
from collections import OrderedDict

import torch

from msamp.common.dtype import Dtypes


class ModelState:
    """Singleton holder (``msamp.nn.model_state``)."""
    def __init__(self):
        self._ready_to_scale_tensor = False
        self._flattened_scaling_metas = None
        self._local_scaling_metas = OrderedDict()
        self._use_fp8_ddp = False

    @property
    def ready_to_scale_tensor(self):
        return self._ready_to_scale_tensor

    @ready_to_scale_tensor.setter
    def ready_to_scale_tensor(self, value):
        self._ready_to_scale_tensor = value

    @property
    def flattened_scaling_metas(self):
        return self._flattened_scaling_metas

    @flattened_scaling_metas.setter
    def flattened_scaling_metas(self, value):
        self._flattened_scaling_metas = value

    @property
    def local_scaling_metas(self):
        return self._local_scaling_metas

    @property
    def use_fp8_ddp(self):
        return self._use_fp8_ddp

    @use_fp8_ddp.setter
    def use_fp8_ddp(self, value):
        self._use_fp8_ddp = value

    def clear(self):
        """Forget every registered meta (used between tests and when a model is rebuilt)."""
        self.__init__()

    @staticmethod
    def _check_in_mem(inner, outer):
        a0 = inner.data_ptr()
        a1 = a0 + inner.numel() * Dtypes.dtype_to_size[inner.dtype]
        b0 = outer.data_ptr()
        b1 = b0 + outer.numel() * Dtypes.dtype_to_size[outer.dtype]
        if inner.device != outer.device or not (b0 <= a0 and a1 <= b1):
            raise RuntimeError(f'Memory ({a0}, {a1}) not in ({b0}, {b1})')

    @staticmethod
    def _flat_tensors(tensors):
        """Pack ``tensors`` into one buffer and re-point each of them at its slice."""
        flat = torch.cat([t.detach().reshape(-1) for t in tensors])
        off = 0
        for t in tensors:
            n = t.numel()
            t.data = flat[off:off + n].view(t.shape)
            off += n
        return flat

    @classmethod
    def _flatten_scaling_metas(cls, metas):
        n = len(metas)
        window = metas[0].window_size
        qtype = metas[0].qtype
        if any(m.window_size != window for m in metas):
            raise RuntimeError('All metas must have the same window_size.')
        if any(m.qtype != qtype for m in metas):
            raise RuntimeError('All metas must have the same qtype.')
        scales = cls._flat_tensors([m.scale for m in metas])
        scales_inv = cls._flat_tensors([m.scale_inv for m in metas])
        amaxs = cls._flat_tensors([m.amax for m in metas])
        counters = cls._flat_tensors([m.amax_counter for m in metas])
        for m in metas:
            m.locked = True
        return dict(qtype=qtype, scales=scales, scales_inv=scales_inv, amaxs=amaxs.view(n, window), amax_counters=counters)

    def rebase(self, key, field, storage):
        """Move the flat buffer ``field`` of meta kind ``key`` into ``storage`` (same dtype and size, e.g. symmetric
        memory) and re-point every registered meta at it; values are preserved."""
        flat = self._flattened_scaling_metas[key]
        old = flat[field]
        new = storage.view(old.shape)
        new.copy_(old)
        attr = {'scales': 'scale', 'scales_inv': 'scale_inv', 'amaxs': 'amax', 'amax_counters': 'amax_counter'}[field]
        for i, metas in enumerate(self._local_scaling_metas.values()):
            t = getattr(metas[key], attr)
            t.data = new[i].view(t.shape)
        flat[field] = new

    def index_of(self, scaling_metas):
        """Position of a layer's meta dict in the flat buffers (registration order), or -1."""
        for i, metas in enumerate(self._local_scaling_metas.values()):
            if metas is scaling_metas:
                return i
        return -1

    def check_metas_in_flat(self, scaling_metas):
        """Raise if a layer's metas no longer alias the flat buffers."""
        if self._flattened_scaling_metas is None:
            return
        for k, v in scaling_metas.items():
            flat = self._flattened_scaling_metas[k]
            self._check_in_mem(v.scale, flat['scales'])
            self._check_in_mem(v.scale_inv, flat['scales_inv'])
            self._check_in_mem(v.amax, flat['amaxs'])
            self._check_in_mem(v.amax_counter, flat['amax_counters'])

    def register_scaling_metas(self, model, group=None):
        """Collect ``scaling_metas`` of every submodule of ``model`` and (re)build the flat buffers."""
        for name, mod in model.named_modules():
            metas = getattr(mod, 'scaling_metas', None)
            if not metas:
                continue
            if any(metas is m for m in self._local_scaling_metas.values()):
                continue
            key, i = name, 2
            while key in self._local_scaling_metas:
                key = f'{name}_{i}'
                i += 1
            self._local_scaling_metas[key] = metas
        all_metas = self.reflatten()
        for metas in all_metas:
            for m in metas.values():
                m.group = group
            self.check_metas_in_flat(metas)

    def reflatten(self):
        """Rebuild the flat buffers from the current tensors of every registered meta (values kept).  Also the way back
        for metas whose tensors were moved elsewhere (e.g. into symmetric memory that is about to be freed)."""
        all_metas = list(self._local_scaling_metas.values())
        if all_metas:
            self._flattened_scaling_metas = {k: self._flatten_scaling_metas([m[k] for m in all_metas]) for k in all_metas[0].keys()}
        return all_metas


model_state = ModelState()
