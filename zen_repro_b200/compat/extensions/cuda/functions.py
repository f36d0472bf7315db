"""``sparse_balance`` and ``hash_index`` with the reference's signatures (extensions/cuda/functions.py:4-15).

``sparse_balance(tensor, memory, serial_memory, partitions, rehash)`` fills the open-addressing table
``memory`` (int32, zero on entry) and the per-partition overflow ``serial_memory`` with element indices
of the nonzeros of ``tensor``.  Differences from the reference, all on purpose: any of fp32 / bf16 / fp16
is accepted (it asserts bf16), slots are claimed atomically so no index is lost under collisions, the
overflow cursor is bounded, and indices are stored **plus one** so that element 0 can be represented
(0 stays the empty-slot sentinel).  ``hash_index(index, partitions)`` writes each position's owner under
the reference's cubic polynomial hash.  CPU tensors run a sequential PyTorch restatement.
"""
from __future__ import annotations

import ctypes

import torch

from .... import _native
from ....sparse import hashing


def sparse_balance(tensor, memory, serial_memory, partitions, rehash=3):
    assert memory.dtype == torch.int32 and serial_memory.dtype == torch.int32
    flat = tensor.reshape(-1)
    msize = memory.numel()
    per_serial = serial_memory.numel() // partitions if partitions else 0
    if not tensor.is_cuda:
        idx = torch.nonzero(flat, as_tuple=True)[0]
        per = msize // partitions
        cursors = [0] * partitions
        for i in idx.tolist():
            first = int(hashing.zen_poly3(torch.tensor([i]), hashing.ZEN_SEEDS[0])) % msize
            part, start = first // per, (first // per) * per
            probes = [first] + [start + int(hashing.zen_poly3(torch.tensor([i]), s)) % per
                                for s in hashing.ZEN_SEEDS[1:max(1, min(rehash, 3))]]
            for s in probes:
                if memory[s] == 0:
                    memory[s] = i + 1
                    break
            else:
                if cursors[part] < per_serial:
                    serial_memory[part * per_serial + cursors[part]] = i + 1
                    cursors[part] += 1
        return
    cursors = torch.zeros(partitions, dtype=torch.int32, device=tensor.device)
    status = torch.zeros(1, dtype=torch.int32, device=tensor.device)
    rc = _native.lib().zen_sparse_balance(_native.ptr(flat), ctypes.c_uint64(flat.numel()), _native.DTYPE_CODE[flat.dtype],
                                          _native.ptr(memory), ctypes.c_uint32(msize), _native.ptr(serial_memory),
                                          ctypes.c_uint32(per_serial), _native.ptr(cursors), partitions, rehash,
                                          _native.ptr(status), _native.stream_ptr())
    _native.check(rc, "zen_sparse_balance")
    return status


def hash_index(index: torch.Tensor, partitions: int):
    """In place: index[i] = owner of position i (``(h(i) % n) // (n // P)`` with ``n = index.numel() // P * P``)."""
    n = index.numel()
    table = max(partitions, n // partitions * partitions)
    if not index.is_cuda:
        index.copy_(hashing.zen_poly3_owner(torch.arange(n), table, partitions).to(index.dtype))
        return index
    assert index.dtype == torch.int32
    from ....sparse.engine import perm_struct
    from ....sparse.hashing import BlockPermutation

    ps = perm_struct(BlockPermutation.make(max(n, 1), partitions, 64))
    rc = _native.lib().zen_owner_map(_native.ptr(index), ctypes.c_uint64(n), ctypes.byref(ps), 1, ctypes.c_uint32(table),
                                     partitions, _native.stream_ptr())
    _native.check(rc, "zen_owner_map")
    return index
