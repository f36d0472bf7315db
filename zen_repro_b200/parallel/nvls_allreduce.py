"""Dense bucket all-reduce through the NVSwitch (``csrc/multimem_allreduce.cu``).

``MulticastArena`` owns one multicast-mapped symmetric region per process group (torch symmetric memory): the
reducer carves its gradient buckets out of it, and ``allreduce_`` reduces a byte range of it in place with the
``multimem.ld_reduce`` / ``multimem.st`` kernel on the current stream, using a capped number of CTAs so that backward
keeps the rest of the GPU.  The call counter lives on the device (bumped by a one-thread kernel before every call), so
a captured step replays correctly.  Replaces, on the data-parallel path, the NCCL all-reduce that torch DDP issues for
the reference (train.py:184-185).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _native
from ..runtime.symmetric import TorchSymmetric

MAX_RANKS = 8
FLAG_BYTES = 256                      # two exchanges x eight sources x four bytes, rounded up


class _McArCtx(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int32), ("nranks", ctypes.c_int32), ("epoch", ctypes.c_uint32), ("pad", ctypes.c_uint32),
                ("wait_ns", ctypes.c_uint64), ("mc", ctypes.c_void_p), ("flags", ctypes.c_void_p * MAX_RANKS),
                ("epoch_dev", ctypes.c_void_p), ("status", ctypes.c_void_p), ("done", ctypes.c_void_p)]


class MulticastArena:
    """``nbytes`` of peer-visible, multicast-mapped device memory (zero-filled) plus the flags of the all-reduce kernel."""

    def __init__(self, nbytes: int, group=None, wait_ms: float = 30000.0, ctas: int | None = None):
        import os

        ctas = ctas if ctas is not None else int(os.environ.get("ZEN_NVLS_CTAS", "16"))
        self.group = group if group is not None else dist.group.WORLD
        self.data_bytes = (nbytes + 255) // 256 * 256
        self.region = TorchSymmetric(self.data_bytes + FLAG_BYTES, self.group)
        if not self.region.multicast_ptr:
            raise RuntimeError("the fabric offers no multicast mapping for this group")
        lib = _native.lib()
        assert lib.zen_mc_ar_ctx_size() == ctypes.sizeof(_McArCtx), "multimem all-reduce ctx layout mismatch"
        dev = self.region._t.device
        self.tensor = self.region._t[: self.data_bytes]                 # uint8 view: buckets are typed slices of it
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._done = torch.zeros(1, dtype=torch.int32, device=dev)
        self._epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        c = _McArCtx()
        c.rank, c.nranks, c.wait_ns = self.region.rank, self.region.nranks, int(wait_ms * 1e6)
        c.mc = self.region.multicast_ptr
        for r in range(self.region.nranks):
            c.flags[r] = self.region.ptrs[r] + self.data_bytes
        c.epoch_dev, c.status, c.done = self._epoch.data_ptr(), self.status.data_ptr(), self._done.data_ptr()
        self.ctx, self.ctas = c, ctas

    def view(self, byte_off: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        es = torch.empty(0, dtype=dtype).element_size()
        return self.tensor[byte_off: byte_off + numel * es].view(dtype)

    def allreduce_(self, byte_off: int, nbytes: int, dtype: torch.dtype, scale: float = 1.0) -> None:
        """Sum over the group (times ``scale``) of the same byte range on every rank, in place, on the current stream."""
        lib = _native.lib()
        _native.check(lib.zen_sparse_epoch_bump(_native.ptr(self._epoch), _native.stream_ptr()), "zen_sparse_epoch_bump")
        rc = lib.zen_multimem_allreduce(ctypes.byref(self.ctx), ctypes.c_uint64(byte_off), ctypes.c_uint64(nbytes),
                                        _native.DTYPE_CODE[dtype], ctypes.c_float(scale), self.ctas, _native.stream_ptr())
        _native.check(rc, "zen_multimem_allreduce")

    def check(self) -> int:
        v = int(self.status.item())
        if v:
            self.status.zero_()
        return v
