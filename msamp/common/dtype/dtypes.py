"""Quantised type tags.

FP8 payloads are carried in byte tensors: ``torch.fp8e4m3`` is ``torch.uint8`` and
``torch.fp8e5m2`` is ``torch.int8``.  The integer values of the tags follow the
numbering used by the reference (msamp/common/dtype/dtypes.py:28-36) because they are
pickled inside checkpoints.
"""
from dataclasses import dataclass

import torch

torch.fp8e4m3 = torch.uint8
torch.fp8e5m2 = torch.int8


@dataclass
class QType:
    """A named quantised type; hashable and convertible to int by its value."""
    name: str
    value: int

    def __int__(self):
        return self.value

    def __hash__(self):
        return self.value


class Dtypes:
    """Namespace with the known quantised types and the torch dtype maps."""
    kbyte = QType('kByte', 0)
    kint32 = QType('kInt32', 1)
    kfloat32 = QType('kFloat32', 2)
    kfloat16 = QType('kFloat16', 3)
    kbfloat16 = QType('kBFloat16', 4)
    kfloat8_e4m3 = QType('kFloat8E4M3', 5)
    kfloat8_e5m2 = QType('kFloat8E5M2', 6)

    dtype_to_qtype = {
        torch.float16: kfloat16,
        torch.bfloat16: kbfloat16,
        torch.float32: kfloat32,
        torch.uint8: kfloat8_e4m3,
        torch.int8: kfloat8_e5m2,
    }
    qtype_to_dtype = {q: d for d, q in dtype_to_qtype.items()}
    dtype_to_size = {
        torch.float32: 4,
        torch.float16: 2,
        torch.bfloat16: 2,
        torch.uint8: 1,
        torch.int8: 1,
        torch.int64: 8,
        torch.int32: 4,
    }
    # torch's own float8 dtypes, used to view byte payloads for emulation and for cuBLASLt.
    qtype_to_float8 = {kfloat8_e4m3: torch.float8_e4m3fn, kfloat8_e5m2: torch.float8_e5m2}

    @classmethod
    def is_fp8_qtype(cls, qtype):
        """True for the two 8-bit floating formats."""
        return qtype.value in (5, 6)

    @classmethod
    def get_dtype_from_qtype(cls, qtype):
        """Storage dtype of a qtype; both FP8 formats are stored as ``torch.uint8``."""
        if cls.is_fp8_qtype(qtype):
            return torch.uint8
        return cls.qtype_to_dtype[qtype]
