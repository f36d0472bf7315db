"""Process-group bootstrap from the torchrun environment (one process per GPU).

Equivalent of ``colossalai.launch_from_torch()`` used by the reference (train.py:109): reads RANK /
LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT, binds the process to its GPU and initialises NCCL
(gloo when no GPU is present, which is how the CPU tests run).
"""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def launch_from_torch(backend: str | None = None, timeout_s: float = 600.0) -> tuple[int, int, torch.device]:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local % torch.cuda.device_count())
        device = torch.device(f"cuda:{torch.cuda.current_device()}")
    else:
        device = torch.device("cpu")
    if not dist.is_initialized():
        kw = dict(backend=backend or ("nccl" if use_cuda else "gloo"), rank=rank, world_size=world,
                  timeout=datetime.timedelta(seconds=timeout_s))
        if use_cuda:
            kw["device_id"] = device
        dist.init_process_group(**kw)
    return rank, world, device
