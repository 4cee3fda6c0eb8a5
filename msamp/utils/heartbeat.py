"""Host-side failure detection for training ranks.

Each rank periodically writes a counter into the job's key-value store (the same ``torch.distributed``
store that bootstrapped the process group); before launching a step a rank can check that every peer has
been seen recently and raise ``RankFailure`` instead of entering a collective that would never complete.
Device-side waits inside the fused kernels are bounded separately and report through the device status
word; together with checkpoint / resume this is the recovery story (there is no in-flight elasticity).
"""
import threading
import time


class RankFailure(RuntimeError):
    """A peer stopped sending heartbeats, or a device-side wait gave up."""


class Heartbeat:
    """Background heartbeat writer plus ``check()`` for stale peers.

    Args:
        store: a ``torch.distributed.Store`` (TCPStore / FileStore / HashStore).
        rank, world: this rank's index and the number of ranks.
        interval: seconds between beats.  timeout: seconds after which a silent peer counts as failed.
    """
    def __init__(self, store, rank, world, interval=1.0, timeout=10.0, prefix='msamp_hb'):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self._stop = threading.Event()
        self._thread = None
        self._last_seen = {}
        self._last_change = {}
        self.beat()

    def _key(self, r):
        return f'{self.prefix}/{r}'

    def beat(self):
        self.store.set(self._key(self.rank), str(time.time()))

    def start(self):
        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:
                    return

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval)

    def stale_ranks(self):
        """Ranks whose heartbeat value has not changed for longer than ``timeout``."""
        now = time.time()
        stale = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = self.store.get(self._key(r)).decode() if self.store.check([self._key(r)]) else None
            except Exception:
                val = None
            if val is None:
                first = self._last_change.setdefault(r, now)
                if now - first > self.timeout:
                    stale.append(r)
                continue
            if self._last_seen.get(r) != val:
                self._last_seen[r] = val
                self._last_change[r] = now
            elif now - self._last_change.get(r, now) > self.timeout:
                stale.append(r)
        return stale

    def check(self, device_status=None):
        """Raise ``RankFailure`` if a peer is stale or ``device_status`` (from ``msamp.ops.native.device_status``) is non-zero."""
        stale = self.stale_ranks()
        if stale:
            raise RankFailure(f'no heartbeat from ranks {stale} for more than {self.timeout} s')
        if device_status:
            raise RankFailure(f'a device-side wait gave up (status bits {device_status:#x}); a peer is late or gone')
