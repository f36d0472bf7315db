"""Host-side failure detection: a heartbeat through the process group's key-value store.

Every rank bumps a counter in the store from a background thread; ``Heartbeat.lost()`` names the ranks whose counter
has not moved for ``timeout`` seconds, judged by this rank's own clock (no clock agreement needed).  A trainer that
calls ``assert_alive()`` between steps learns of a departed peer on the host, before it launches kernels or collectives
that would wait for that peer; the device-side waits are bounded as well, this is the cheaper first line.  The
reference has neither (it relies on NCCL's watchdog, comm.py / DDPbackend.py have no timeouts).
"""
from __future__ import annotations

import threading
import time

import torch.distributed as dist


class PeerLost(RuntimeError):
    def __init__(self, ranks):
        super().__init__(f"no heartbeat from rank(s) {sorted(ranks)}")
        self.ranks = sorted(ranks)


class Heartbeat:
    def __init__(self, interval: float = 0.5, timeout: float = 5.0, store=None, rank: int | None = None,
                 world: int | None = None, prefix: str = "zen_hb"):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = dist.PrefixStore(prefix, store)
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.interval, self.timeout = interval, timeout
        self._beats = 0
        self._stop = threading.Event()
        self._seen = {}                      # rank -> (last counter value, local time it last changed)
        self._beat()                         # the key exists before anyone reads it
        self._thread = threading.Thread(target=self._run, name="zen-heartbeat", daemon=True)
        self._thread.start()

    def _beat(self):
        self._beats += 1
        self.store.set(f"r{self.rank}", str(self._beats))

    def _run(self):
        while not self._stop.wait(self.interval):
            try:
                self._beat()
            except Exception:                # the store went away with the job
                return

    def stop(self):
        """Stop beating (a rank that leaves between steps calls this, or simply exits)."""
        self._stop.set()
        self._thread.join(timeout=2 * self.interval + 1.0)

    def lost(self) -> list:
        """Ranks whose heartbeat has been silent for longer than ``timeout`` seconds."""
        now = time.monotonic()
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = int(self.store.get(f"r{r}"))
            except Exception:
                val = -1
            last = self._seen.get(r)
            if last is None or last[0] != val:
                self._seen[r] = (val, now)
            elif now - last[1] > self.timeout:
                out.append(r)
        return out

    def assert_alive(self):
        gone = self.lost()
        if gone:
            raise PeerLost(gone)
