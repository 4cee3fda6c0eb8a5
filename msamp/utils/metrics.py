"""Step metrics as JSON lines: tokens/s, peak memory, per-phase milliseconds, skipped steps, scale statistics."""
import json
import time

import torch


class StepMetrics:
    """Append one JSON object per logged step to ``path`` (or keep them in memory when ``path`` is None)."""
    def __init__(self, path=None, rank=0):
        self.path, self.rank = path, rank
        self.records = []
        self.skipped_steps = 0
        self._t_last = time.perf_counter()

    def log(self, step, tokens=None, loss=None, phases=None, **extra):
        now = time.perf_counter()
        rec = {'step': step, 'rank': self.rank, 'wall_s': now - self._t_last, 'skipped_steps': self.skipped_steps}
        self._t_last = now
        if tokens is not None and rec['wall_s'] > 0:
            rec['tokens_per_s'] = tokens / rec['wall_s']
        if loss is not None:
            rec['loss'] = float(loss)
        if torch.cuda.is_available():
            rec['peak_mem_gib'] = torch.cuda.max_memory_allocated() / 2**30
        if phases:
            rec['phases_ms'] = phases
        rec.update(extra)
        self.records.append(rec)
        if self.path:
            with open(self.path, 'a') as f:
                f.write(json.dumps(rec) + '\n')
        return rec

    @staticmethod
    def scale_histogram():
        """Per-kind (input / wgrad / ograd) log2-scale statistics of every registered FP8 layer."""
        from msamp.nn import model_state
        flat = model_state.flattened_scaling_metas
        if not flat:
            return {}
        out = {}
        for kind, bufs in flat.items():
            s = torch.log2(bufs['scales'].float().clamp_min(1e-30)).cpu()
            out[kind] = {'min_log2': float(s.min()), 'max_log2': float(s.max()), 'mean_log2': float(s.mean()), 'layers': int(s.numel())}
        return out
