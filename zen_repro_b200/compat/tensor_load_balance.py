"""``TensorPartition`` with the reference's surface (tensor_load_balance.py:5-51).

``load_balance(tensor) -> (indices[P], values[P], splits)`` assigns every nonzero of a flat tensor to one of
``partitions`` owners.  Two partitioners: ``hash="perm"`` (default) is this framework's invertible block
permutation, evaluated with tensor ops; ``hash="zen_poly3"`` reproduces the reference's table-based balancer
through the ``sparse_balance`` kernel (probes inside the partition chosen by the first hash, overflow list
per partition).  Indices are int32 element indices, position 0 included.
"""
from __future__ import annotations

import torch

from ..sparse.hashing import BlockPermutation
from ..utils.trace import trace_range
from .extensions.cuda.functions import sparse_balance


class TensorPartition:
    def __init__(self, partitions: int, memory_scale: int = 1, rehash: int = 3, hash: str = "perm", block: int = 64):
        self.partitions, self.memory_scale, self.rehash, self.hash, self.block = partitions, memory_scale, rehash, hash, block

    # -- reference-compatible table path ---------------------------------------------------------
    def balance_sparse_tensor(self, tensor):
        numel, P = tensor.numel(), self.partitions
        msize = max(P, int(numel * self.memory_scale) // P * P)
        memory = torch.zeros(msize, dtype=torch.int32, device=tensor.device)
        serial = torch.zeros(max(P, numel // P // 10 * P), dtype=torch.int32, device=tensor.device)
        with trace_range("balance_sparse_tensor"):
            sparse_balance(tensor, memory, serial, P, rehash=self.rehash)
        return memory, serial

    def get_sub_sparse_tensors(self, tensor, memory):
        flat = tensor.reshape(-1)
        idx_l, val_l, splits = [], [], []
        with trace_range("get_sub_sparse_tensors"):
            for chunk in memory.chunk(self.partitions):
                idx = chunk[chunk != 0] - 1                       # stored +1, see sparse_balance
                idx_l.append(idx)
                val_l.append(flat[idx.long()])
                splits.append(idx.numel())
        return idx_l, val_l, splits

    def load_balance(self, tensor):
        flat = tensor.reshape(-1)
        P = self.partitions
        if self.hash == "zen_poly3":
            memory, serial = self.balance_sparse_tensor(flat)
            i1, v1, s1 = self.get_sub_sparse_tensors(flat, memory)
            i2, v2, s2 = self.get_sub_sparse_tensors(flat, serial)
            idx = [torch.cat([a, b]) for a, b in zip(i1, i2)]
            val = [torch.cat([a, b]) for a, b in zip(v1, v2)]
            splits = torch.tensor([a + b for a, b in zip(s1, s2)], device=flat.device)
            return idx, val, splits
        perm = BlockPermutation.make(flat.numel(), P, self.block)
        nz = torch.nonzero(flat, as_tuple=True)[0]
        owner, _ = perm.owner_slot(nz)
        idx, val = [], []
        for p in range(P):
            m = owner == p
            idx.append(nz[m].to(torch.int32))
            val.append(flat[nz[m]])
        splits = torch.tensor([i.numel() for i in idx], device=flat.device)
        return idx, val, splits
