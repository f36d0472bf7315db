"""Symmetric (peer-visible) device memory.

Every rank allocates one region of the same size; each rank ends up with a
table of ``P`` base pointers, its own and its peers', that kernels index by
rank to load from or store into another GPU's memory over NVLink.

Providers:

``LocalSymmetric``   ``P`` regions on ONE device.  Used to run all ranks of a
                     collective phase by phase on a single GPU (tests, P = 1).
``IpcSymmetric``     one process per GPU; regions come from ``cudaMalloc`` and
                     their CUDA IPC handles are exchanged through
                     ``torch.distributed`` (object all-gather over the group).
``TorchSymmetric``   the same table obtained from
                     ``torch.distributed._symmetric_memory`` (adds a multicast
                     address when the fabric offers one).

The reference has no counterpart: it moves every byte through NCCL calls issued
from Python (DDPbackend.py:14-81).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _native


class SymmetricRegion:
    """Base: ``ptrs[r]`` is the address of rank ``r``'s region as seen from this rank."""

    rank: int
    nranks: int
    nbytes: int
    ptrs: list[int]
    multicast_ptr: int = 0

    def local_ptr(self) -> int:
        return self.ptrs[self.rank]

    def view(self, rank: int, offset: int, nbytes: int, dtype: torch.dtype) -> torch.Tensor:
        """A tensor aliasing ``nbytes`` at ``offset`` of rank ``rank``'s region (debug / tests)."""
        esz = torch.empty(0, dtype=dtype).element_size()

        class _Arr:
            pass

        a = _Arr()
        a.__cuda_array_interface__ = {
            "shape": (nbytes // esz,), "typestr": {1: "|u1", 2: "<u2", 4: "<u4", 8: "<u8"}[esz],
            "data": (self.ptrs[rank] + offset, False), "version": 2,
        }
        raw = torch.as_tensor(a, device=f"cuda:{torch.cuda.current_device()}")
        return raw.view(dtype)

    def close(self) -> None:
        pass


class LocalSymmetric:
    """``P`` regions on the current device; ``for_rank(r)`` gives rank ``r``'s view of the table."""

    def __init__(self, nranks: int, nbytes: int, device=None):
        self.nranks, self.nbytes = nranks, nbytes
        self.device = torch.device(device or f"cuda:{torch.cuda.current_device()}")
        self._bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=self.device) for _ in range(nranks)]
        self.ptrs = [b.data_ptr() for b in self._bufs]

    def for_rank(self, rank: int) -> SymmetricRegion:
        r = SymmetricRegion()
        r.rank, r.nranks, r.nbytes, r.ptrs = rank, self.nranks, self.nbytes, list(self.ptrs)
        r._keep = self._bufs
        return r


class IpcSymmetric(SymmetricRegion):
    def __init__(self, nbytes: int, group=None):
        lib = _native.lib()
        self.group = group
        self.rank = dist.get_rank(group)
        self.nranks = dist.get_world_size(group)
        self.nbytes = nbytes
        base = ctypes.c_void_p()
        _native.check(lib.zen_sym_alloc(ctypes.byref(base), ctypes.c_uint64(nbytes)), "zen_sym_alloc")
        self._own = base.value
        h = (ctypes.c_ubyte * 64)()
        _native.check(lib.zen_ipc_get_handle(ctypes.c_void_p(self._own), h), "zen_ipc_get_handle")
        mine = (bytes(h), torch.cuda.current_device(), os.getpid())
        everyone: list = [None] * self.nranks
        dist.all_gather_object(everyone, mine, group=group)
        self.ptrs, self._opened = [], []
        for r, (handle, dev, pid) in enumerate(everyone):
            if r == self.rank:
                self.ptrs.append(self._own)
                continue
            if pid == os.getpid():
                raise RuntimeError("IpcSymmetric needs one process per rank")
            p = ctypes.c_void_p()
            hb = (ctypes.c_ubyte * 64).from_buffer_copy(handle)
            _native.check(lib.zen_ipc_open(hb, ctypes.byref(p)), f"zen_ipc_open(rank {r})")
            self.ptrs.append(p.value)
            self._opened.append(p.value)
        dist.barrier(group=group)

    def close(self) -> None:
        lib = _native.lib()
        for p in self._opened:
            lib.zen_ipc_close(ctypes.c_void_p(p))
        self._opened = []
        if self._own and self.nranks > 1 and dist.is_initialized():
            # every peer has unmapped this rank's region before it is freed
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        if self._own:
            lib.zen_sym_free(ctypes.c_void_p(self._own))
            self._own = 0


class TorchSymmetric(SymmetricRegion):
    def __init__(self, nbytes: int, group=None):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.nranks = dist.get_world_size(self.group)
        self.nbytes = nbytes
        self._t = symm.empty(nbytes, dtype=torch.uint8, device=f"cuda:{torch.cuda.current_device()}")
        self._t.zero_()
        self._hdl = symm.rendezvous(self._t, self.group.group_name)
        self.ptrs = [int(p) for p in self._hdl.buffer_ptrs]
        self.multicast_ptr = int(getattr(self._hdl, "multicast_ptr", 0) or 0)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)


def make_symmetric(nbytes: int, group=None, backend: str | None = None) -> SymmetricRegion:
    """Region for this process's rank in ``group`` (``ZEN_SYMM_BACKEND`` = ``ipc`` | ``torch``)."""
    backend = backend or os.environ.get("ZEN_SYMM_BACKEND", "ipc")
    if backend == "torch":
        return TorchSymmetric(nbytes, group)
    return IpcSymmetric(nbytes, group)
