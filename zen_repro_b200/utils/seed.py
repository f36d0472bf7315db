"""Seeding of every RNG a run touches (python, numpy, torch CPU and CUDA), as utils.py:33-38 of the reference."""
import random

import numpy as np
import torch


def set_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    try:
        import transformers

        transformers.set_seed(seed)
    except Exception:
        pass
