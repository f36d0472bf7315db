"""Functional ops: each has a CUDA kernel path (sm_100a) and a PyTorch reference used on CPU and in tests."""
from .elementwise import (act_bwd, act_fwd, colsum, cross_entropy, embedding_bwd_rows, embedding_fwd,  # noqa: F401
                          norm_bwd, norm_fwd, rope_, rows_add_)
