"""Named phase timers (CUDA events on GPU, wall clock on CPU) and NVTX ranges.

The phase names used by the engines match the ones the reference inherits from DeepSpeed / Megatron
(``overflow_check, compute_norm, unscale_and_clip, basic_step, update_fp16, optimizer_allgather,
optimizer_gradients, optimizer_step`` – msamp/deepspeed/runtime/fp8/fused_optimizer.py:192-260,
zero/fp8_stage_1_and_2.py:667-670) so existing log parsers keep working.
"""
import contextlib
import time

import torch


@contextlib.contextmanager
def nvtx_range(name):
    """NVTX range when CUDA is available, otherwise a no-op."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class _Phase:
    def __init__(self, name, use_cuda):
        self.name, self.use_cuda = name, use_cuda
        self.pending = []
        self.total_ms, self.count = 0.0, 0
        self._t0 = None

    def start(self):
        if self.use_cuda:
            self._t0 = torch.cuda.Event(enable_timing=True)
            self._t0.record()
        else:
            self._t0 = time.perf_counter()

    def stop(self):
        if self._t0 is None:
            return
        if self.use_cuda:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            self.pending.append((self._t0, e1))
        else:
            self.total_ms += (time.perf_counter() - self._t0) * 1e3
        self.count += 1
        self._t0 = None

    def flush(self):
        """Fold finished event pairs into the total without blocking on unfinished ones."""
        keep = []
        for e0, e1 in self.pending:
            if e1.query():
                self.total_ms += e0.elapsed_time(e1)
            else:
                keep.append((e0, e1))
        self.pending = keep


class PhaseTimers:
    """``timers('name').start() / .stop()``, ``with timers.phase('name')``, ``timers.log(names)``."""
    def __init__(self, enabled=True):
        self.enabled = enabled
        self.phases = {}
        self.use_cuda = torch.cuda.is_available()

    def __call__(self, name):
        if name not in self.phases:
            self.phases[name] = _Phase(name, self.use_cuda)
        return self.phases[name]

    @contextlib.contextmanager
    def phase(self, name):
        if not self.enabled:
            yield
            return
        with nvtx_range(name):
            p = self(name)
            p.start()
            try:
                yield
            finally:
                p.stop()

    def summary(self, reset=False, synchronize=False):
        """``{name: mean milliseconds}`` of the finished measurements."""
        if synchronize and self.use_cuda:
            torch.cuda.synchronize()
        out = {}
        for name, p in self.phases.items():
            p.flush()
            done = p.count - len(p.pending)
            out[name] = p.total_ms / done if done else 0.0
            if reset:
                p.total_ms, p.count, p.pending = 0.0, 0, []
        return out

    def log(self, names=None, logger=None, reset=True):
        s = self.summary(reset=reset, synchronize=True)
        text = ' | '.join(f'{k}: {v:.2f} ms' for k, v in s.items() if names is None or k in names)
        if logger is not None:
            logger.info(text)
        return text
