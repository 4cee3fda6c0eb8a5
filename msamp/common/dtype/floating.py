"""Largest finite value of each floating format (reference: msamp/common/dtype/floating.py:17-53)."""
import torch

from msamp.common.dtype.dtypes import Dtypes


class Floating:
    """Tables of maximum finite magnitudes keyed by torch dtype and by qtype."""
    fp_maxs = {}
    qfp_max = {}

    @staticmethod
    def _get_fp_max(exp, man, inf_existed=True):
        """Largest finite value of a binary float with ``exp`` exponent and ``man`` mantissa bits.

        With ``inf_existed`` the all-ones exponent is reserved (IEEE style); without it only the
        all-ones mantissa of that exponent is reserved for NaN, which is the e4m3 "fn" variant.
        """
        bias = 2**(exp - 1) - 1
        if inf_existed:
            top_exp = (2**exp - 2) - bias
            frac = 2.0 - 2.0**(-man)
        else:
            top_exp = (2**exp - 1) - bias
            frac = 2.0 - 2.0**(1 - man)
        return float(frac * 2.0**top_exp)


_E4M3 = Floating._get_fp_max(4, 3, inf_existed=False)
_E5M2 = Floating._get_fp_max(5, 2)
_F16 = Floating._get_fp_max(5, 10)
_BF16 = Floating._get_fp_max(8, 7)
_F32 = Floating._get_fp_max(8, 23)
Floating.fp_maxs = {torch.uint8: _E4M3, torch.int8: _E5M2, torch.float16: _F16, torch.bfloat16: _BF16, torch.float32: _F32}
Floating.qfp_max = {
    Dtypes.kfloat8_e4m3: _E4M3,
    Dtypes.kfloat8_e5m2: _E5M2,
    Dtypes.kfloat16: _F16,
    Dtypes.kbfloat16: _BF16,
    Dtypes.kfloat32: _F32,
}
