"""Per-rank logger: file ``{rank}.log`` (truncated at start) plus stdout, lines prefixed ``[rank{r}]: time - msg``
(same sinks and format as the reference's ``setup_logger``, train.py:28-54)."""
from __future__ import annotations

import logging
import os
import sys

import torch.distributed as dist


def setup_logger(log_dir: str = ".", to_stdout: bool = True, level=logging.INFO) -> logging.Logger:
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    logger = logging.getLogger(f"rank_{rank}_logger")
    logger.setLevel(level)
    logger.propagate = False
    for h in list(logger.handlers):
        logger.removeHandler(h)
    fmt = logging.Formatter(f"[rank{rank}]: %(asctime)s - %(message)s")
    os.makedirs(log_dir, exist_ok=True)
    fh = logging.FileHandler(os.path.join(log_dir, f"{rank}.log"), "w")
    fh.setFormatter(fmt)
    logger.addHandler(fh)
    if to_stdout:
        sh = logging.StreamHandler(sys.stdout)
        sh.setFormatter(fmt)
        logger.addHandler(sh)
    return logger
