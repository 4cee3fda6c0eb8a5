"""GPU identification.

The reference enables FP8 GEMM only when the device name contains "h100"
(msamp/common/utils/device.py:18-22).  Here FP8 tensor-core GEMM is available on any device of
compute capability 10.x (tcgen05); other CUDA devices are rejected by the native kernels.
"""
from enum import Enum

import torch


def default_device():
    """Device on which converted modules and new metas are placed.

    The current CUDA device when one is visible, otherwise the CPU.  ``MSAMP_DEVICE=cpu`` pins the
    CPU emulation even on a GPU machine (used by the gloo multi-process tests).
    """
    import os
    forced = os.environ.get('MSAMP_DEVICE')
    if forced:
        return torch.device(forced)
    if torch.cuda.is_available():
        return torch.device('cuda', torch.cuda.current_device())
    return torch.device('cpu')


class GPUType(Enum):
    """Vendor of the visible accelerator."""
    NVIDIA = 1
    AMD = 2
    UNKNOWN = 3


class Device:
    """Static queries about the current accelerator."""
    @staticmethod
    def get_gpu_type():
        if not torch.cuda.is_available():
            return GPUType.UNKNOWN
        return GPUType.AMD if getattr(torch.version, 'hip', None) else GPUType.NVIDIA

    @staticmethod
    def is_blackwell(index=None):
        if not torch.cuda.is_available():
            return False
        return torch.cuda.get_device_capability(index)[0] == 10

    @staticmethod
    def is_fp8_supported():
        """FP8 GEMM runs natively on sm_100; on CPU it is emulated, so the answer is always yes."""
        return True
