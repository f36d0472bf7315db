"""Status words of the communication kernels, mirrored to the host without a synchronisation in the hot loop.

The sparse engines and the fused tensor-parallel GEMMs never fault on a missing peer or a full slot: they set bits
in a device status word and return (the reference's NCCL path blocks instead, DDPbackend.py:44-46).  Somebody has to
read those words.  ``StatusMirror`` does it one step late:

* ``publish()`` (every step, after the gradient synchronisation, on the current stream): gather the words into one
  small device vector, MAX-all-reduce it over the data-parallel group so that every rank holds the same value, bump a
  sequence number and copy vector + sequence number into pinned host memory.  All of it is stream-ordered device work
  (it can be captured in a CUDA graph); the host does not wait.
* ``poll()`` (start of the next step): wait, normally not at all, until the copy of the step before the last one has
  landed and return the agreed value.  Every rank therefore learns of a failure at the same step and can take the
  same recovery action there (``Trainer`` re-broadcasts the replicas and switches the failing path to its library
  form).

Bits: 1 record overflow, 2 gather overflow, 4 wait expired, 8 overflow reported by a peer, 16 bad argument.
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist


class SyncStatusError(RuntimeError):
    pass


def decode(bits: int) -> str:
    names = [(1, "record slot overflow"), (2, "gather payload overflow"), (4, "a wait on a peer expired"),
             (8, "a peer reported overflow"), (16, "bad argument")]
    return ", ".join(n for b, n in names if bits & b) or "ok"


class StatusMirror:
    def __init__(self, device, group=None, lag: int = 1, wait_s: float = 30.0):
        self.device, self.group, self.lag, self.wait_s = torch.device(device), group, lag, wait_s
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.sources: list[tuple[str, torch.Tensor]] = []
        self._dev = None
        self._host = None
        self.published = 0
        self._clean_from = 0               # publishes before this number predate the last clear() and are ignored
        self.last: dict[str, int] = {}

    def add(self, name: str, word: torch.Tensor) -> None:
        """Register a one-element int32 status word (before the first ``publish``)."""
        assert self._dev is None, "sources are fixed once publishing has started"
        self.sources.append((name, word))

    RING = 4          # per-step slots, so that every rank reads the value of the same step whatever has landed since

    def _ensure(self):
        if self._dev is None:
            n = len(self.sources)
            self._dev = torch.zeros(n + 1, dtype=torch.int32, device=self.device)         # [statuses..., sequence number]
            self._ring = torch.zeros(self.RING, n + 1, dtype=torch.int32, device=self.device)
            self._host = torch.zeros(self.RING, n + 1, dtype=torch.int32)
            if self.device.type == "cuda":
                self._host = self._host.pin_memory()

    def publish(self) -> None:
        self._ensure()
        n = len(self.sources)
        if n:
            torch.cat([w.reshape(1).to(torch.int32) for _, w in self.sources], out=self._dev[:n])
            if self.world > 1:
                dist.all_reduce(self._dev[:n], op=dist.ReduceOp.MAX, group=self.group)
        self._dev[n:] += 1
        slot = torch.remainder(self._dev[n:], self.RING).long()           # stays on the device: replayable in a graph
        self._ring.index_copy_(0, slot, self._dev.unsqueeze(0))
        self._host.copy_(self._ring, non_blocking=True)
        self.published += 1

    def poll(self) -> dict[str, int]:
        """Agreed status per source as of publish number ``published - lag`` (empty dict = clean).  Identical on every
        rank: the words were MAX-reduced on the device and every rank reads the slot of the same step."""
        if self._dev is None or self.published <= self.lag:
            return {}
        need = self.published - self.lag
        if need < self._clean_from:
            return {}
        n = len(self.sources)
        row = self._host[need % self.RING]
        t0 = time.monotonic()
        while int(row[n]) != need:
            if int(row[n]) > need:
                raise SyncStatusError(f"status slot of step {need} was overwritten (host ran {self.RING} steps behind)")
            if time.monotonic() - t0 > self.wait_s:
                raise SyncStatusError(f"status copy of step {need} did not arrive within {self.wait_s} s")
            time.sleep(50e-6)
        vals = [int(row[i]) for i in range(n)]
        self.last = {name: v for (name, _), v in zip(self.sources, vals) if v}
        return dict(self.last)

    def clear(self) -> None:
        """Zero the device words (after a recovery), in stream order."""
        for _, w in self.sources:
            w.zero_()
        self._clean_from = self.published + 1
