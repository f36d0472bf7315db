"""Master-rank helpers (``DistCoordinator`` of the reference's training script, train.py:110,186,203,216-220)."""
from __future__ import annotations

import torch.distributed as dist


class DistCoordinator:
    def __init__(self):
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world_size = dist.get_world_size() if dist.is_initialized() else 1

    def is_master(self) -> bool:
        return self.rank == 0

    def print_on_master(self, msg: str) -> None:
        if self.is_master():
            print(msg, flush=True)

    def block_all(self) -> None:
        if dist.is_initialized():
            dist.barrier()
