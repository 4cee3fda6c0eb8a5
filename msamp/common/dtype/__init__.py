"""Quantised-type enumeration and floating-point range tables."""
from msamp.common.dtype.dtypes import Dtypes, QType
from msamp.common.dtype.floating import Floating

__all__ = ['Dtypes', 'QType', 'Floating']
