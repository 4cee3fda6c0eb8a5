"""ctypes loader for the sm_100a kernel library."""
import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'libmsamp_b200.so')

_lib = None
_lock = threading.Lock()

# dtype codes shared with csrc/common.cuh
DT_F32, DT_F16, DT_BF16 = 0, 1, 2
_DT = {torch.float32: DT_F32, torch.float16: DT_F16, torch.bfloat16: DT_BF16}
FMT_E4M3, FMT_E5M2 = 0, 1

_ERRORS = {
    1: 'invalid argument',
    2: 'unsupported dtype',
    3: 'CUDA launch failure',
    4: 'device wait timed out',
    5: 'tensor map encode failed',
    6: 'size exceeds static scratch capacity',
    7: 'device is not sm_100',
}


class NativeError(RuntimeError):
    """A native entry point returned a non-zero status."""


def dt(dtype):
    """dtype code of a high-precision torch dtype."""
    try:
        return _DT[dtype]
    except KeyError:
        raise TypeError(f'unsupported dtype for native kernels: {dtype}') from None


def fmt(qtype):
    """FP8 format code of a qtype (5 = e4m3, 6 = e5m2)."""
    return FMT_E4M3 if int(qtype) == 5 else FMT_E5M2


def available():
    """True if the native library file exists (it may still fail to load without a driver)."""
    return os.path.exists(LIB_PATH)


def lib():
    """Load (once) and return the native library; raise if it cannot be used."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f'{LIB_PATH} is missing: build it with `python -m msamp.ops.build` '
                        '(CUDA tensors never fall back to the CPU emulation)'
                    )
                handle = ctypes.CDLL(LIB_PATH)
                handle.msamp_last_error.restype = ctypes.c_char_p
                _lib = handle
    return _lib


launch_count = 0    # native entry points called so far (each launches at least one kernel)


def check(status, what=''):
    """Raise ``NativeError`` for a non-zero status code; counts the call."""
    global launch_count
    launch_count += 1
    if status != 0:
        detail = lib().msamp_last_error().decode()
        raise NativeError(f'{what}: {_ERRORS.get(status, status)} ({detail})')


_raw_stream = getattr(torch._C, '_cuda_getCurrentRawStream', None)
_raw_device = getattr(torch._C, '_cuda_getDevice', None)


def stream():
    """Raw handle of torch's current CUDA stream (called once per launch, so it avoids the Python stream objects)."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    """Device pointer of a tensor (None → NULL)."""
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def i64(v):
    return ctypes.c_int64(int(v))


def ctypes_float(v):
    return ctypes.c_float(float(v))


def peek_device_status():
    """The device-side error word without clearing it (no synchronisation: the word lives in mapped host memory)."""
    fn = getattr(lib(), 'msamp_peek_device_status', None)
    return int(fn()) if fn is not None else 0


def device_status():
    """Read and clear the device-side error word (non-zero after a bounded wait gave up)."""
    return lib().msamp_read_device_status()
