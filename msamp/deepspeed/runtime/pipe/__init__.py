"""Pipeline-parallel engine."""
from msamp.deepspeed.runtime.pipe.engine import MSAMPPipelineEngine, PipelineModule

__all__ = ['MSAMPPipelineEngine', 'PipelineModule']
