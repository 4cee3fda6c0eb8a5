"""Logging, lazy import, process-group and device helpers."""
from msamp.common.utils.logging import MsAmpLogger, logger
from msamp.common.utils.lazy_import import LazyImport
from msamp.common.utils.dist import DistUtil
from msamp.common.utils.device import Device, GPUType

TransformerEngineWrapper = LazyImport('msamp.common.utils.transformer_engine_wrapper', 'TransformerEngineWrapper')

__all__ = ['MsAmpLogger', 'logger', 'LazyImport', 'DistUtil', 'Device', 'GPUType', 'TransformerEngineWrapper']
