"""``LoadBalanceAllreduce`` with the reference's surface (comm.py:8-146).

``zen_sparse_comm(tensor, method)`` returns the dense element-wise SUM over the process group of the
(already sparsified) inputs: method 1 = sparse all-gather of COO, 2 = balanced exchange + COO gather,
3 = balanced exchange + hash-bitmap gather.  CUDA tensors run the fused P2P engine
(``sparse/engine.py``); CPU tensors, or ``transport="library"``, run the same algorithm over
``torch.distributed`` collectives.  The helper methods of the reference class are kept with their
meanings (element indices instead of table contents; bitmaps LSB-first over the caller's owned slots).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..sparse import formats, torch_pipeline
from ..sparse.hashing import BlockPermutation
from ..utils.trace import trace_range
from .DDPbackend import DDPBackend
from .tensor_load_balance import TensorPartition


class LoadBalanceAllreduce:
    def __init__(self, process_group, global_ranks=None, logger=None, memory_scale=1, rehash=3, *, block: int = 64,
                 transport: str = "auto", max_density: float = 0.12, deterministic: bool = False):
        self.name = "LoadBalanceAllreduce"
        self.ddp = DDPBackend(process_group, global_ranks, logger)
        self.process_group = process_group
        self.partitions = dist.get_world_size(process_group)
        self.local_rank = dist.get_rank(group=process_group)
        self.logger = logger
        self.block, self.transport, self.max_density, self.deterministic = block, transport, max_density, deterministic
        self.tensor_partition = self.get_tensor_partition_obj(memory_scale, rehash)
        self.mapping: dict = {}
        self._engines: dict = {}

    def get_tensor_partition_obj(self, memory_scale, rehash):
        return TensorPartition(partitions=self.partitions, memory_scale=memory_scale, rehash=rehash, block=self.block)

    # ---- helpers kept from the reference class ----------------------------------------------------
    def stack_tensors(self, tensors, shape=-1):
        return (torch.cat(list(tensors)) if isinstance(tensors, (list, tuple)) else tensors).reshape(shape)

    def encode_sparse_tensor(self, tensor):
        return formats.coo_encode(tensor)

    def decode_sparse_tensors(self, indices_tensors, values_tensors, alltoall_dense_size):
        idx = self.stack_tensors(indices_tensors)
        val = self.stack_tensors(values_tensors)
        return formats.coo_decode(idx, val, alltoall_dense_size)

    def calculate_mapping(self, numel):
        """Per-owner ascending position lists under the block permutation (arithmetic, but materialised here
        because the reference API returns lists)."""
        perm = BlockPermutation.make(numel, self.partitions, self.block)
        owner, _ = perm.owner_slot(torch.arange(numel))
        return [torch.nonzero(owner == p, as_tuple=True)[0] for p in range(self.partitions)]

    def encode_bitmap(self, sparse_indices, numel):
        if numel not in self.mapping:
            self.mapping[numel] = self.calculate_mapping(numel)
        own = self.mapping[numel][self.local_rank].to(sparse_indices.device)
        mask = torch.zeros(own.numel(), dtype=torch.bool, device=own.device)
        mask[torch.searchsorted(own, sparse_indices)] = True
        return formats.pack_bitmap(mask)

    def decode_bitmap(self, bitmap_indices, numel):
        if numel not in self.mapping:
            self.mapping[numel] = self.calculate_mapping(numel)
        out = []
        for p, bm in enumerate(bitmap_indices):
            own = self.mapping[numel][p].to(bm.device)
            out.append(own[formats.unpack_bitmap(bm, own.numel())])
        return out

    # ---- the collective ----------------------------------------------------------------------------
    def _engine(self, numel: int):
        eng = self._engines.get(numel)
        if eng is None:
            from ..sparse.engine import SparseAllReduce

            eng = SparseAllReduce(numel, self.process_group, block=self.block, max_density=self.max_density,
                                  methods=(1, 2, 3), deterministic=self.deterministic)
            self._engines[numel] = eng
        return eng

    def zen_sparse_comm(self, tensor, method):
        if self.partitions == 1:
            return tensor
        use_cuda = tensor.is_cuda and self.transport in ("auto", "p2p")
        with trace_range(f"zen_sparse_comm_m{method}"):
            if use_cuda:
                return self._engine(tensor.numel())(tensor.contiguous(), method=method)
            return torch_pipeline.dist_sparse_allreduce(tensor, self.process_group, method=method, block=self.block)

    def check(self) -> int:
        """OR of the status words of every engine used so far (0 = ok); synchronises."""
        st = 0
        for e in self._engines.values():
            st |= e.check()
        return st
