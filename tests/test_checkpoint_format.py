"""Checkpoint format: module paths, class names and attribute names of pickled ScalingTensors are shared with the reference.

The first test unpickles a stream that was assembled opcode by opcode from the reference's documented layout
(msamp/common/tensor/tensor.py:72-91, 132-138; meta.py:27-35; hook.py; dtypes.py:14-17) - not produced by this
library's classes - and loads it into a model and an optimizer.  The second checks the other direction: what this
library pickles carries no attribute outside that layout.
"""
import pickle

import torch

import msamp
from msamp.common.dtype import Dtypes
from msamp.common.tensor import ScalingMeta, ScalingTensor

ST_ATTRS = {'value', 'meta', '_grad', '_backward_post_hooks', '_requires_grad'}
META_ATTRS = {'qtype', 'scale', 'scale_inv', 'amax', 'amax_counter', 'window_size', 'group', 'locked'}
HOOK_ATTRS = {'hooks', 'history_counter'}


def _frag(obj):
    """Pickle opcodes that push ``obj`` (protocol 2 stream without its header and STOP)."""
    return pickle.dumps(obj, protocol=2)[2:-1]


def _instance(module, cls, state):
    """Opcodes that build ``module.cls`` by NEWOBJ and BUILD it from ``state`` (attribute name -> opcode fragment)."""
    out = b'c' + module.encode() + b'\n' + cls.encode() + b'\n' + b')' + b'\x81' + b'}' + b'('
    for key, frag in state.items():
        out += _frag(key) + frag
    return out + b'u' + b'b'


def _reference_scaling_tensor(value, qtype_name, qtype_value, scale, window=1, scale_as_float=False):
    qtype = _instance('msamp.common.dtype.dtypes', 'QType', {'name': _frag(qtype_name), 'value': _frag(qtype_value)})
    s = torch.tensor(float(scale))
    meta = _instance('msamp.common.tensor.meta', 'ScalingMeta', {
        'qtype': qtype,
        'scale': _frag(float(scale)) if scale_as_float else _frag(s),    # after a CUDA step the reference leaves a Python float here
        'scale_inv': _frag(1.0 / float(scale)) if scale_as_float else _frag(s.reciprocal()),
        'amax': _frag(torch.zeros(window)), 'amax_counter': _frag(torch.zeros((), dtype=torch.int32)), 'window_size': _frag(window),
        'group': _frag(None), 'locked': _frag(False)})
    hooks = _instance('msamp.common.tensor.hook', 'HookManager', {'hooks': _frag({}), 'history_counter': _frag(0)})
    return _instance('msamp.common.tensor.tensor', 'ScalingTensor', {
        'value': _frag(value), 'meta': meta, '_grad': _frag(None), '_backward_post_hooks': hooks, '_requires_grad': _frag(False)})


def _stream(fragment):
    return b'\x80\x02' + fragment + b'.'


def test_reference_shaped_pickles_load_into_model_and_optimizer():
    torch.manual_seed(0)
    w = torch.randn(4, 16) * 0.1
    scale = 2.0**12
    value = (w * scale).half()    # O2 weight: scaled fp16
    st = pickle.loads(_stream(_reference_scaling_tensor(value, 'kFloat16', 3, scale)))
    assert isinstance(st, ScalingTensor) and isinstance(st.meta, ScalingMeta) and st.meta.qtype == Dtypes.kfloat16
    assert set(st.__dict__) == ST_ATTRS and set(st.meta.__dict__) == META_ATTRS
    assert torch.allclose(st.float(), w, atol=1e-3)
    # a model state dict with that entry
    model = torch.nn.Sequential(torch.nn.Linear(16, 4))
    model = msamp.nn.LinearReplacer.replace(model)
    sd = model.state_dict()
    sd['0.weight'] = st
    model.load_state_dict(sd)
    assert torch.allclose(model[0].weight.float(), w, atol=1e-3)
    # optimizer state with e4m3 / fp16 moments whose metas carry Python-float scales (reference quirk after a CUDA step)
    opt = msamp.optim.LBAdamW(model.parameters(), lr=1e-3, exp_avg_dtype=torch.uint8, exp_avg_sq_dtype=torch.float16)
    model(torch.randn(2, 16)).sum().backward()
    opt.step()
    own = opt.state_dict()
    m8 = (torch.randn(4, 16) * 8).to(torch.float8_e4m3fn).view(torch.uint8)
    v16 = (torch.rand(4, 16) * 100).half()
    exp_avg = pickle.loads(_stream(_reference_scaling_tensor(m8, 'kFloat8E4M3', 5, 64.0, scale_as_float=True)))
    exp_avg_sq = pickle.loads(_stream(_reference_scaling_tensor(v16, 'kFloat16', 3, 1024.0, scale_as_float=True)))
    idx = own['param_groups'][0]['params'][0]
    own['state'][idx] = {'step': 7, 'exp_avg': exp_avg, 'exp_avg_sq': exp_avg_sq}
    opt.load_state_dict(own)
    state = opt.state[model[0].weight]
    assert int(state['step']) == 7
    assert torch.allclose(state['exp_avg'].float(), m8.view(torch.float8_e4m3fn).float() / 64.0)
    assert torch.allclose(state['exp_avg_sq'].float(), v16.float() / 1024.0)
    model(torch.randn(2, 16)).sum().backward()
    opt.step()    # the loaded state is usable


def _walk(obj, seen):
    if isinstance(obj, ScalingTensor):
        seen.append(obj)
    elif isinstance(obj, dict):
        for v in obj.values():
            _walk(v, seen)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            _walk(v, seen)


def test_own_pickles_carry_only_the_shared_attribute_set():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.Linear(32, 4))
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    model, opt = msamp.initialize(model, opt, 'O2')
    for _ in range(2):    # run-time attributes (FP8 weight cache, gradients) get attached to the live parameters here
        opt.zero_grad()
        model(torch.randn(8, 16)).sum().backward()
        opt.step()
    for blob in (model.state_dict(), opt.state_dict()):
        restored = pickle.loads(pickle.dumps(blob))
        found = []
        _walk(restored, found)
        assert found
        for st in found:
            assert set(st.__dict__) <= ST_ATTRS, set(st.__dict__) - ST_ATTRS
            assert set(st.meta.__dict__) <= META_ATTRS, set(st.meta.__dict__) - META_ATTRS
            assert set(st._backward_post_hooks.__dict__) <= HOOK_ATTRS
            assert type(st).__module__ == 'msamp.common.tensor.tensor' and type(st.meta).__module__ == 'msamp.common.tensor.meta'
            assert type(st.meta.qtype).__module__ == 'msamp.common.dtype.dtypes'
