"""The push protocol of the CUDA sparse engine, restated on CPU ranks with a key-value store as the "peer memory".

What the GPU engine does with P2P stores and flag words (``csrc/sparse_kernels.cu``) happens here with the same
phases and the same failure semantics, so that the host-visible behaviour can be tested without a GPU and with
faults injected on the host:

  phase 1  every rank partitions its non-zeros by owner and PUSHES (slots, values) into the owner's inbox, then
           publishes a mail ``(count, info, epoch)``; more records than the inbox holds -> the sender truncates and
           sets REC_OVERFLOW in the mail (the bit travels, so the receiver knows too)
  phase 2  the owner WAITS, bounded, for the mail of every source -> TIMEOUT when one does not arrive; reduces
  phase 3  the owner pushes (bitmap | COO, values) to every peer and publishes a mail per peer
  phase 4  every rank waits, bounded, for every owner's mail and densifies

Statuses use the bits of the CUDA engine (1 record overflow, 2 gather overflow, 4 wait expired, 8 overflow seen at a
peer).  ``EmulatedSparseAllReduce`` then agrees on the status with one MAX all-reduce and, when it is not zero, falls
back to the dense all-reduce of the original tensor, the same recovery the training hook applies: the step still gets a
correct gradient and the caller sees which bits were raised.  ``faults`` injects, per rank: "mute" (the rank skips its
pushes of a phase), "slow" (sleeps before pushing), "short" (publishes a mail that claims fewer records than it sent
space for, as a torn write would).  The reference has no such path (comm.py has no timeouts or capacity checks).
"""
from __future__ import annotations

import io
import time

import torch
import torch.distributed as dist

from . import torch_pipeline as TP
from .hashing import BlockPermutation

REC_OVERFLOW, GATHER_OVERFLOW, TIMEOUT, PEER_OVERFLOW = 1, 2, 4, 8


def _dumps(obj) -> bytes:
    b = io.BytesIO()
    torch.save(obj, b)
    return b.getvalue()


def _loads(raw: bytes):
    return torch.load(io.BytesIO(raw), weights_only=False)


class EmulatedSparseAllReduce:
    def __init__(self, numel: int, group=None, *, max_density: float = 0.12, wait_s: float = 2.0, block: int = 64,
                 store=None, faults: dict | None = None):
        self.group = group
        self.P = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.numel = numel
        self.perm = BlockPermutation.make(numel, self.P, block)
        # inbox capacity per (source -> owner), as the CUDA plan sizes it: the expected share plus slack
        self.cap_rec = max(16, int(numel * max_density / self.P * 1.5))
        self.cap_gather = max(16, int(self.perm.slots_per_part * min(1.0, max_density * self.P)))
        self.wait_s = wait_s
        base = store if store is not None else dist.distributed_c10d._get_default_store()
        self.store = dist.PrefixStore("zen_emul", base)
        self.epoch = 0
        self.faults = faults or {}
        self.last_status = 0
        self.last_fallback = False

    # ---- "peer memory" ------------------------------------------------------------------------------------------
    def _push(self, phase: str, dst: int, payload, count: int, info: int):
        key = f"{phase}/{self.epoch}/{self.rank}->{dst}"
        self.store.set(key + "/data", _dumps(payload))
        self.store.set(key + "/mail", _dumps((count, info, self.epoch)))      # the mail goes last, like the release store

    def _wait(self, phase: str, src: int):
        """Bounded wait for the mail src -> this rank; returns (payload, count, info) or None when it expired."""
        key = f"{phase}/{self.epoch}/{src}->{self.rank}"
        deadline = time.monotonic() + self.wait_s
        while not self.store.check([key + "/mail"]):
            if time.monotonic() > deadline:
                return None
            time.sleep(0.005)
        count, info, epoch = _loads(self.store.get(key + "/mail"))
        if epoch != self.epoch:
            return None
        return _loads(self.store.get(key + "/data")), count, info

    def _fault(self, kind: str):
        v = self.faults.get(kind)
        if v is None:
            return None
        if isinstance(v, dict):
            return v.get(self.rank)
        return True if self.rank in v else None

    # ---- one call -----------------------------------------------------------------------------------------------
    def __call__(self, tensor: torch.Tensor, method: int = 3) -> torch.Tensor:
        self.epoch += 1
        flat = tensor.reshape(-1)
        status = 0
        fmt = "bitmap" if method == 3 else "coo"
        slots, vals, counts = TP.partition(flat, self.perm)
        slow = self._fault("slow")
        if slow:
            time.sleep(float(slow))
        # phase 1: push records to their owners
        if not self._fault("mute"):
            for o in range(self.P):
                n, info = counts[o], 0
                if n > self.cap_rec:
                    n, info = self.cap_rec, REC_OVERFLOW
                    status |= REC_OVERFLOW
                claimed = max(0, n - 3) if self._fault("short") else n
                self._push("rec", o, (slots[o][:n], vals[o][:n]), claimed, info)
        # phase 2: owner side
        rs, rv = [], []
        for s in range(self.P):
            got = self._wait("rec", s)
            if got is None:
                status |= TIMEOUT
                continue
            (sl, vl), count, info = got
            if info & REC_OVERFLOW:
                status |= PEER_OVERFLOW
            if count != sl.numel():                 # a mail that does not match what arrived: treat as lost records
                status |= PEER_OVERFLOW
                sl, vl = sl[:count], vl[:count]
            rs.append(sl)
            rv.append(vl)
        acc = TP.owner_reduce(rs, rv, self.perm.slots_per_part)
        payload, gvals = TP.gather_encode(acc, fmt, tensor.dtype)
        ginfo = 0
        if gvals.numel() > self.cap_gather:
            ginfo = GATHER_OVERFLOW
            status |= GATHER_OVERFLOW
        # phase 3: push the reduced slice to every peer
        if not self._fault("mute"):
            for p in range(self.P):
                self._push("gat", p, (payload, gvals), int(gvals.numel()), ginfo | (status & (REC_OVERFLOW | PEER_OVERFLOW | TIMEOUT)))
        # phase 4: densify
        oslots, ovals = [], []
        for o in range(self.P):
            got = self._wait("gat", o)
            if got is None:
                status |= TIMEOUT
                oslots.append(torch.zeros(0, dtype=torch.int64))
                ovals.append(torch.zeros(0, dtype=tensor.dtype))
                continue
            (pl, gv), count, info = got
            if info:
                status |= PEER_OVERFLOW if info & (REC_OVERFLOW | PEER_OVERFLOW | GATHER_OVERFLOW) else 0
                status |= TIMEOUT if info & TIMEOUT else 0
            oslots.append(TP.gather_decode(pl, fmt, self.perm.slots_per_part))
            ovals.append(gv)
        out = TP.densify(oslots, ovals, self.perm, tensor.dtype).reshape(tensor.shape)
        # every rank must take the same decision: agree on the status, then fall back collectively if needed
        st = torch.tensor([status], dtype=torch.int64)
        dist.all_reduce(st, op=dist.ReduceOp.BOR if hasattr(dist.ReduceOp, "BOR") else dist.ReduceOp.MAX, group=self.group)
        self.last_status = int(st.item())
        self.last_fallback = self.last_status != 0
        if self.last_fallback:
            out = tensor.clone()
            dist.all_reduce(out, group=self.group)
        return out
