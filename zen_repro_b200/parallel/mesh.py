"""DP x TP process-group mesh.

World ranks are laid out with the tensor-parallel coordinate innermost (``rank = dp * tp_size + tp``):
tensor-parallel peers are neighbouring GPUs, and a data-parallel group is the set of ranks with equal
TP coordinate.  Mirrors what the reference reads from ColossalAI's plugin: ``model.dp_group``,
``model.tp_group`` and ``plugin.pg_mesh.get_ranks_in_group`` (train.py:162-166, 177).
"""
from __future__ import annotations

import torch.distributed as dist


class ProcessGroupMesh:
    def __init__(self, tp_size: int = 1, pp_size: int = 1, backend: str | None = None):
        if pp_size != 1:
            raise NotImplementedError("pipeline parallelism is not part of this framework (pp_size must be 1)")
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        if self.world % tp_size:
            raise ValueError(f"world size {self.world} is not a multiple of tp_size {tp_size}")
        self.tp_size, self.dp_size = tp_size, self.world // tp_size
        self.tp_rank, self.dp_rank = self.rank % tp_size, self.rank // tp_size
        self._ranks: dict = {}
        self.tp_group = self.dp_group = None
        if not dist.is_initialized():
            return
        # every rank creates every group, in the same order
        for d in range(self.dp_size):
            ranks = [d * tp_size + t for t in range(tp_size)]
            g = dist.new_group(ranks, backend=backend)
            self._ranks[id(g)] = ranks
            if d == self.dp_rank:
                self.tp_group = g
        for t in range(tp_size):
            ranks = [d * tp_size + t for d in range(self.dp_size)]
            g = dist.new_group(ranks, backend=backend)
            self._ranks[id(g)] = ranks
            if t == self.tp_rank:
                self.dp_group = g

    def get_ranks_in_group(self, group) -> list[int]:
        if group is None:
            return list(range(self.world))
        return list(self._ranks[id(group)])

    def coordinate(self) -> dict:
        return {"dp": self.dp_rank, "tp": self.tp_rank}
