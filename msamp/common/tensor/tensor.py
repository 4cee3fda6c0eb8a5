"""ScalingTensor: a low-precision payload plus its ScalingMeta, with a tensor-like surface.

It is deliberately a plain object (not a ``torch.Tensor`` subclass), like the reference's
(msamp/common/tensor/tensor.py:15-660): pickled checkpoints contain instances of
``msamp.common.tensor.tensor.ScalingTensor`` whose attribute names (``value``, ``meta``, ``_grad``,
``_backward_post_hooks``, ``_requires_grad``) are therefore part of the file format.

Importing this module also teaches a few torch entry points about ScalingTensor
(``Tensor.cast``, ``Tensor.fused_cast_transpose``, ``Tensor.qtype``, ``zeros_like``, ``ones_like``,
``overrides.is_tensor_like``, ``is_floating_point`` and the AMP unscale/inf-check primitive).
"""
import torch
import torch.nn.functional as F

from msamp.common.dtype import Dtypes
from msamp.common.tensor.hook import HookManager
from msamp.common.tensor.meta import ScalingMeta
from msamp.common.tensor.cast import TypeCast
from msamp.ops import cast as _k

_HP_DTYPES = (torch.float32, torch.float16, torch.bfloat16)


class ScalingTensor:
    """``value`` (uint8 FP8 bytes, or fp16/bf16/fp32 scaled data) interpreted through ``meta``."""
    def __init__(self, value, meta):
        expected = Dtypes.get_dtype_from_qtype(meta.qtype)
        if expected != value.dtype:
            raise TypeError(f'Type mismatch, value.dtype is {value.dtype}, meta.dtype is {expected} (meta.qtype is {meta.qtype}).')
        self.value = value
        self._grad = None
        self._backward_post_hooks = HookManager()
        self.meta = meta
        self._requires_grad = False

    # ---- autograd-like surface -----------------------------------------------------------------
    @property
    def grad(self):
        return self._grad

    @grad.setter
    def grad(self, grad):
        self._grad = grad

    @grad.deleter
    def grad(self):
        self._grad = None

    @property
    def requires_grad(self):
        return self._requires_grad

    @requires_grad.setter
    def requires_grad(self, flag):
        self._requires_grad = bool(flag)

    def requires_grad_(self, requires_grad=True):
        self._requires_grad = bool(requires_grad)
        return self

    @property
    def grad_fn(self):
        return None

    @property
    def is_leaf(self):
        return True

    def register_backward_post_hook(self, fn):
        """``fn(manager, (grad,), grad)`` runs each time ``backward_grad_update`` delivers a gradient."""
        return self._backward_post_hooks.register_hook(fn)

    def backward_grad_update(self, grad):
        """Store ``grad`` and fire the post-backward hooks (used instead of autograd for weight gradients)."""
        self._grad = grad
        self._backward_post_hooks(grad)

    def detach(self):
        """A new ScalingTensor sharing value and meta, without grad or hooks."""
        return ScalingTensor(self.value, self.meta)

    # ---- conversions ---------------------------------------------------------------------------
    def _dequant(self, otype):
        q = self.meta.qtype
        if Dtypes.is_fp8_qtype(q):
            return TypeCast.cast_from_fp8(self.value, self.meta, otype)
        if q in (Dtypes.kfloat16, Dtypes.kbfloat16, Dtypes.kfloat32):
            return TypeCast.cast_from_fp16(self.value, self.meta, otype)
        raise TypeError(f'Unsupported Type: {q}')

    def float(self):
        return self._dequant(Dtypes.kfloat32)

    def half(self):
        return self._dequant(Dtypes.kfloat16)

    def bfloat16(self):
        return self._dequant(Dtypes.kbfloat16)

    def to(self, *args, **kwargs):
        """``to(dtype)`` dequantises to a torch.Tensor; ``to(device)`` moves this ScalingTensor."""
        dtype, device, non_blocking = None, None, False
        names = {torch.dtype: 'dtype', torch.device: 'device', bool: 'non_blocking', str: 'device'}
        seen = set()
        items = [(names.get(type(a)), a) for a in args if a is not None] + [(k, v) for k, v in kwargs.items() if v is not None]
        for name, val in items:
            if name is None or name not in ('dtype', 'device', 'non_blocking'):
                raise TypeError(f'Unsupported argument for ScalingTensor.to: {val!r}')
            if name in seen:
                raise TypeError(f'Duplicated argument: {name}')
            seen.add(name)
            if name == 'dtype':
                dtype = val
            elif name == 'device':
                device = torch.device(val)
            else:
                non_blocking = val
        out = self
        if dtype is not None:
            if dtype == torch.float32:
                out = self.float()
            elif dtype == torch.float16:
                out = self.half()
            elif dtype == torch.bfloat16:
                out = self.bfloat16()
            else:
                raise TypeError(f'unsupported dtype: {dtype}')
        if device is not None:
            if isinstance(out, ScalingTensor):
                out.value = out.value.to(device=device, non_blocking=non_blocking)
                if out.meta.device != out.value.device:
                    if out.meta.locked:
                        raise ValueError('This ScalingTensor is locked.')
                    out.meta.to(device)
            else:
                out = out.to(device=device, non_blocking=non_blocking)
        return out

    def cast(self, qtype):
        """Re-quantise to ``qtype`` reusing the stored amax (no pass over the data to find it)."""
        if qtype == self.meta.qtype:
            return self
        if Dtypes.is_fp8_qtype(self.meta.qtype):
            return self.float().cast(qtype)
        # value == x * old_scale; we want x * new_scale where new_scale comes from amax(x).
        meta = ScalingMeta(qtype, amax=self.meta.amax.clone(), window_size=self.meta.window_size, device=self.value.device)
        meta.reset_scaling_factor()
        true_scale_inv = torch.reciprocal(meta.scale)
        meta.scale.mul_(self.meta.scale_inv)    # factor that maps the stored value to the new payload
        if Dtypes.is_fp8_qtype(qtype):
            value = _k.cast_to_fp8(self.value.contiguous(), qtype, meta.scale)
        else:
            value = (self.value.float() * meta.scale).to(Dtypes.get_dtype_from_qtype(qtype))
        meta.scale.copy_(torch.reciprocal(true_scale_inv))
        meta.scale_inv.copy_(true_scale_inv)
        return ScalingTensor(value, meta)

    def cast_(self, qtype):
        if self.qtype == qtype:
            return self
        e = self.cast(qtype)
        self.value.data = e.value
        self.meta.qtype = e.meta.qtype
        self.meta.scale.copy_(e.meta.scale)
        self.meta.scale_inv.copy_(e.meta.scale_inv)
        self.meta.amax.copy_(e.meta.amax)
        return self

    def fp8_transpose(self):
        if not Dtypes.is_fp8_qtype(self.meta.qtype):
            raise TypeError(f'Unsupported FP8 transpose type: {self.meta.qtype}')
        return ScalingTensor(_k.transpose_fp8(self.value.reshape(-1, self.value.shape[-1])), self.meta)

    # ---- scalar arithmetic acts on scale_inv only -----------------------------------------------
    @torch.no_grad()
    def mul_(self, other):
        if torch.is_tensor(other):
            if other.numel() != 1:
                raise ValueError('The tensor must by single-element tensor.')
            other = other.reshape(self.meta.scale_inv.shape).to(self.meta.scale_inv.device)
        self.meta.scale_inv.mul_(other)
        return self

    @torch.no_grad()
    def div_(self, other):
        if torch.is_tensor(other):
            if other.numel() != 1:
                raise ValueError('The tensor must by single-element tensor.')
            other = other.reshape(self.meta.scale_inv.shape).to(self.meta.scale_inv.device)
        self.meta.scale_inv.div_(other)
        return self

    # ---- tensor-like helpers --------------------------------------------------------------------
    def t(self):
        return ScalingTensor(self.value.t(), self.meta)

    def contiguous(self):
        meta = self.meta if self.value.is_contiguous() else self.meta.clone()
        return ScalingTensor(self.value.contiguous(), meta)

    def has_inf_or_nan(self):
        return not bool(torch.isfinite(self.meta.amax[0]))

    def abs(self):
        if self.value.dtype == torch.uint8:
            return ScalingTensor(self.value & 0x7F, self.meta.clone())
        if self.value.dtype not in _HP_DTYPES:
            raise TypeError(f'not support {self.value.dtype}')
        return ScalingTensor(self.value.abs(), self.meta.clone())

    def min(self):
        return self.float().min()

    def max(self):
        return self.float().max()

    def isnan(self):
        if Dtypes.is_fp8_qtype(self.qtype):
            if self.qtype == Dtypes.kfloat8_e4m3:
                return (self.value & 0x7F) == 0x7F
            return (self.value & 0x7F) > 0x7C
        return torch.isnan(self.value)

    def zero_(self):
        self.value.zero_()
        return self

    def flatten(self):
        return ScalingTensor(self.value.flatten(), self.meta)

    def view(self, *shape):
        return ScalingTensor(self.value.view(*shape), self.meta)

    def reshape(self, *shape):
        return ScalingTensor(self.value.reshape(*shape), self.meta)

    def pad(self, pad):
        return ScalingTensor(F.pad(self.value, pad), self.meta)

    def clone(self):
        return ScalingTensor(self.value.clone(), self.meta.clone())

    def cpu(self, *args, **kwargs):
        meta = self.meta.clone().cpu()
        return ScalingTensor(self.value.cpu(), meta)

    def cuda(self, *args, **kwargs):
        self.value = self.value.cuda()
        if not self.meta.is_cuda:
            if self.meta.locked:
                raise ValueError('This ScalingTensor is locked.')
            self.meta.to(self.value.device)
        return self

    def copy_(self, src):
        if not isinstance(src, ScalingTensor):
            raise TypeError(f'The input should be a ScalingTensor rather than {type(src)}')
        with torch.no_grad():
            if self.value.dtype != src.value.dtype:
                raise TypeError('The dtype of value must be same.')
            self.value.copy_(src.value)
            self.meta.copy_(src.meta)
        return self

    @property
    def data(self):
        return self.detach()

    @data.setter
    def data(self, data):
        with torch.no_grad():
            if isinstance(data, ScalingTensor):
                if self.meta.locked and self.meta is not data.meta:
                    raise ValueError('This ScalingTensor is locked.')
                self.value.data = data.value
                self.meta = data.meta
            elif isinstance(data, torch.Tensor):
                self.value.data = data
            else:
                raise TypeError('The type of data is not supported')

    @property
    def qtype(self):
        return self.meta.qtype

    @property
    def dtype(self):
        return self.value.dtype

    @property
    def shape(self):
        return self.value.shape

    @property
    def size(self):
        return self.value.size

    @property
    def device(self):
        return self.value.device

    @property
    def is_cuda(self):
        return self.value.is_cuda

    @property
    def is_meta(self):
        return self.value.is_meta

    @property
    def is_sparse(self):
        return self.value.is_sparse

    @property
    def ndim(self):
        return self.value.dim()

    def dim(self):
        return self.value.dim()

    def numel(self):
        return self.value.numel()

    def nelement(self):
        return self.value.numel()

    def element_size(self):
        return self.value.element_size()

    def data_ptr(self):
        return self.value.data_ptr()

    def stride(self, *a):
        return self.value.stride(*a)

    def type(self):
        return f'{self.__class__.__module__}.{self.__class__.__qualname__}'

    def is_contiguous(self):
        return self.value.is_contiguous()

    def is_floating_point(self):
        return False

    def is_complex(self):
        return False

    def __len__(self):
        return len(self.value)

    def __repr__(self):
        return f'ScalingTensor({self.float()}, meta={self.meta})'

    def __setstate__(self, state):
        self.__dict__.update(state)
        self.__dict__.setdefault('_grad', None)
        self.__dict__.setdefault('_requires_grad', False)
        if '_backward_post_hooks' not in self.__dict__:
            self._backward_post_hooks = HookManager()


class TorchOverider:
    """Installs the torch-side patches listed in the module docstring (idempotent)."""
    one_scales = dict()
    torch_unary_funcs = ['torch.zeros_like', 'torch.ones_like', 'torch.overrides.is_tensor_like']
    _installed = False

    @classmethod
    def override(cls):
        if cls._installed:
            return
        cls._installed = True
        torch.Tensor.cast = cls._cast_to_scalingtensor
        torch.Tensor.fused_cast_transpose = cls._fused_cast_transpose_to_scalingtensors
        torch.Tensor.qtype = property(lambda self: Dtypes.dtype_to_qtype[self.dtype])
        for name in cls.torch_unary_funcs:
            base, attr = cls._get_func_base_and_name(name)
            old = getattr(base, attr)
            setattr(base, attr, cls._wrap(old, lambda x, *a, _old=old, **k: _old(x.value, *a, **k)))
        torch.is_floating_point = cls._wrap(torch.is_floating_point, lambda x: x.is_floating_point())
        torch._amp_foreach_non_finite_check_and_unscale_ = cls._wrap_unscale(torch._amp_foreach_non_finite_check_and_unscale_)

    @staticmethod
    def _cast_to_scalingtensor(self, qtype, meta=None, sync=False):
        """``tensor.cast(qtype, meta=None, sync=False) -> ScalingTensor``."""
        x = self.contiguous()
        if meta is None:
            meta = ScalingMeta(qtype, device=x.device)
        if Dtypes.is_fp8_qtype(qtype):
            return ScalingTensor(TypeCast.cast_to_fp8(x, meta, sync=sync), meta)
        return ScalingTensor(TypeCast.cast_to_fp16(x, meta, sync=sync), meta)

    @staticmethod
    def _fused_cast_transpose_to_scalingtensors(self, qtype, meta=None, sync=False):
        """``tensor.fused_cast_transpose(qtype, ...) -> (ScalingTensor, ScalingTensor transposed)``; FP8 only."""
        if not Dtypes.is_fp8_qtype(qtype):
            raise TypeError(f'Unsupported Cast: {self.dtype} -> {qtype}')
        x = self.contiguous()
        if meta is None:
            meta = ScalingMeta(qtype, device=x.device)
        out, out_t = TypeCast.cast_to_fp8(x, meta, sync=sync, fuse_transpose=True)
        return ScalingTensor(out, meta), ScalingTensor(out_t, meta)

    @staticmethod
    def _get_func_base_and_name(func_name):
        parts = func_name.split('.')
        if len(parts) < 2 or parts[0] != 'torch':
            raise ValueError(f'Invalid function name: {func_name}')
        base = torch
        for e in parts[1:-1]:
            base = getattr(base, e)
        return base, parts[-1]

    @staticmethod
    def _wrap(old_fn, scaling_fn):
        def fn(input, *args, **kwargs):
            if isinstance(input, ScalingTensor):
                return scaling_fn(input, *args, **kwargs)
            return old_fn(input, *args, **kwargs)

        fn.__wrapped__ = old_fn
        return fn

    @classmethod
    def _wrap_unscale(cls, old_fn):
        @torch.no_grad()
        def new_fn(grads, found_inf, inv_scale):
            """Unscale + inf check that treats a ScalingTensor grad through its ``scale_inv`` and ``amax[0]``."""
            cpu_grads, dev_grads, sinv, amax0 = [], [], [], []
            for g in grads:
                if isinstance(g, ScalingTensor):
                    sinv.append(g.meta.scale_inv)
                    amax0.append(g.meta.amax[0])
                elif g.is_cuda:
                    dev_grads.append(g)
                else:
                    cpu_grads.append(g)
            if dev_grads:
                old_fn(dev_grads, found_inf, inv_scale)
            for g in cpu_grads:
                g.mul_(inv_scale.to(g.device))
                if not torch.isfinite(g).all():
                    found_inf.fill_(1.0)
            if sinv:
                if sinv[0].is_cuda:
                    old_fn(sinv, found_inf, inv_scale)
                    dev = found_inf.device
                    if dev not in cls.one_scales:
                        cls.one_scales[dev] = torch.ones(1, device=dev)
                    old_fn(amax0, found_inf, cls.one_scales[dev])
                else:
                    for s, a in zip(sinv, amax0):
                        s.mul_(inv_scale.to(s.device))
                        if not (torch.isfinite(s) and torch.isfinite(a)):
                            found_inf.fill_(1.0)

        new_fn.__wrapped__ = old_fn
        return new_fn


TorchOverider.override()
