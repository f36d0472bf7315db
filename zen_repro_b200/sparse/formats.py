"""Index encodings used on the wire: COO and bitmap (LSB-first).

Bit ``j`` of byte ``k`` of a bitmap stands for slot ``8 k + j`` -- the same
LSB-first packing as the reference (comm.py:76-84 packs with weights
``2**arange(8)``; comm.py:93-95 unpacks with the same weights).
"""
from __future__ import annotations

import torch

_WEIGHTS = None


def _weights(device) -> torch.Tensor:
    return torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.int32, device=device)


def pack_bitmap(mask: torch.Tensor) -> torch.Tensor:
    """bool/uint8 mask[n] -> uint8[ceil(n/8)], LSB-first."""
    n = mask.numel()
    nbytes = (n + 7) // 8
    m = torch.zeros(nbytes * 8, dtype=torch.int32, device=mask.device)
    m[:n] = mask.reshape(-1).to(torch.int32)
    return (m.view(nbytes, 8) * _weights(mask.device)).sum(dim=1).to(torch.uint8)


def unpack_bitmap(bitmap: torch.Tensor, nbits: int) -> torch.Tensor:
    """uint8[nbytes] -> bool[nbits], LSB-first."""
    b = bitmap.to(torch.int32).unsqueeze(-1)
    bits = (b & _weights(bitmap.device)) != 0
    return bits.reshape(-1)[:nbits]


def coo_encode(dense: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Ascending int64 indices of the nonzeros of a flat tensor and their values (comm.py:47-50)."""
    flat = dense.reshape(-1)
    idx = torch.nonzero(flat, as_tuple=True)[0]
    return idx, flat[idx]


def coo_decode(idx: torch.Tensor, val: torch.Tensor, numel: int, dtype=None) -> torch.Tensor:
    """zeros(numel).scatter_add_(idx, val) (comm.py:32-44)."""
    out = torch.zeros(numel, dtype=dtype or val.dtype, device=val.device)
    if idx.numel():
        out.scatter_add_(0, idx.to(torch.int64), val.to(out.dtype))
    return out


def choose_index_format(union_count: int, slots: int, index_bytes: int = 4) -> str:
    """'bitmap' when the bitmap is the smaller encoding of ``union_count`` of ``slots`` positions.

    The bitmap costs ``slots / 8`` bytes whatever the count; COO costs
    ``index_bytes`` per nonzero.  Above roughly 3 % occupancy (int32 indices) the
    bitmap wins; near-full unions fall back to a dense slice.
    """
    if union_count * 2 >= slots:          # values alone exceed half a dense slice: send dense
        return "dense"
    return "bitmap" if union_count * index_bytes * 8 > slots else "coo"
