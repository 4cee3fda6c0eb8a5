"""Runtime utilities: phase timers, NVTX ranges, JSONL step metrics, heartbeat-based failure detection."""
from msamp.utils.timer import PhaseTimers, nvtx_range
from msamp.utils.metrics import StepMetrics
from msamp.utils.heartbeat import Heartbeat, RankFailure

__all__ = ['PhaseTimers', 'nvtx_range', 'StepMetrics', 'Heartbeat', 'RankFailure']
