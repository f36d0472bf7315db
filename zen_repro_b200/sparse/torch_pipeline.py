"""Pure-PyTorch sparse all-reduce: the oracle and the CPU / library transport path.

Stages (each a pure function, each mirrored by one CUDA kernel):

    partition   : nonzeros of the flat bucket -> per-owner (slot, value) records
    exchange    : all-to-all of the records                       (transport)
    owner_reduce: scatter-add records into this owner's S slots (fp32 accumulate)
    gather_enc  : owner slice -> bitmap | COO slots + values in ascending slot order
    exchange    : all-gather of the encodings                      (transport)
    densify     : zero-fill + scatter into the full-length result

Behavioural contract (comm.py:101-146): the result is the element-wise SUM
over ranks of the inputs, method 1 = sparse all-gather of COO, method 2 =
balanced all-to-all + COO gather, method 3 = balanced all-to-all + bitmap
gather.  Unlike the reference, position 0 is transmittable, ``numel % P`` may
be anything, and accumulation is fp32 in fixed source order.

Two drivers: :func:`simulate` runs all ranks in one process (unit tests);
:func:`dist_sparse_allreduce` runs one rank over ``torch.distributed`` (gloo
on CPU -- ``all_to_all_single`` because gloo has no list all-to-all -- or NCCL
as the library baseline).
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from .formats import pack_bitmap, unpack_bitmap
from .hashing import BlockPermutation

# --------------------------------------------------------------------------- stages


def partition(flat: torch.Tensor, perm: BlockPermutation):
    """-> (slots[P] int32 lists, values[P] lists, counts[P]) in ascending element order."""
    idx = torch.nonzero(flat, as_tuple=True)[0]
    val = flat[idx]
    owner, slot = perm.owner_slot(idx)
    slots, vals, counts = [], [], []
    for p in range(perm.parts):
        m = owner == p
        slots.append(slot[m].to(torch.int32))
        vals.append(val[m])
        counts.append(int(m.sum()))
    return slots, vals, counts


def owner_reduce(rec_slots: Sequence[torch.Tensor], rec_vals: Sequence[torch.Tensor], nslots: int) -> torch.Tensor:
    """fp32 accumulator over this owner's slots; sources are added in list order."""
    acc = torch.zeros(nslots, dtype=torch.float32, device=rec_vals[0].device if rec_vals else "cpu")
    for s, v in zip(rec_slots, rec_vals):
        if s.numel():
            acc.index_add_(0, s.to(torch.int64), v.to(torch.float32))
    return acc


def gather_encode(acc: torch.Tensor, fmt: str, out_dtype: torch.dtype):
    """Owner slice -> (index payload, values) with values in ascending slot order."""
    nz = acc != 0
    vals = acc[nz].to(out_dtype)
    if fmt == "bitmap":
        return pack_bitmap(nz), vals
    if fmt == "coo":
        return torch.nonzero(nz, as_tuple=True)[0].to(torch.int32), vals
    raise ValueError(fmt)


def gather_decode(payload: torch.Tensor, fmt: str, nslots: int) -> torch.Tensor:
    """Index payload -> ascending int64 slot list."""
    if fmt == "bitmap":
        return torch.nonzero(unpack_bitmap(payload, nslots), as_tuple=True)[0]
    return payload.to(torch.int64)


def densify(per_owner_slots: Sequence[torch.Tensor], per_owner_vals: Sequence[torch.Tensor],
            perm: BlockPermutation, out_dtype: torch.dtype) -> torch.Tensor:
    dev = per_owner_vals[0].device
    out = torch.zeros(perm.padded_numel, dtype=out_dtype, device=dev)
    for o, (s, v) in enumerate(zip(per_owner_slots, per_owner_vals)):
        if s.numel():
            out[perm.index_of(o, s)] = v.to(out_dtype)
    return out[: perm.numel]


# --------------------------------------------------------------------------- in-process driver


def simulate(inputs: Sequence[torch.Tensor], method: int = 3, block: int = 64) -> list[torch.Tensor]:
    """Run the full pipeline for ``P = len(inputs)`` ranks in one process; returns each rank's result."""
    P = len(inputs)
    shape, dtype = inputs[0].shape, inputs[0].dtype
    flats = [t.reshape(-1) for t in inputs]
    N = flats[0].numel()
    if method == 1:
        acc = torch.zeros(N, dtype=torch.float32, device=flats[0].device)
        for f in flats:                                    # fixed source order
            idx = torch.nonzero(f, as_tuple=True)[0]
            acc.index_add_(0, idx, f[idx].to(torch.float32))
        return [acc.to(dtype).reshape(shape).clone() for _ in range(P)]
    perm = BlockPermutation.make(N, P, block)
    parts = [partition(f, perm) for f in flats]
    fmt = "bitmap" if method == 3 else "coo"
    enc = []
    for o in range(P):
        acc = owner_reduce([parts[s][0][o] for s in range(P)], [parts[s][1][o] for s in range(P)],
                           perm.slots_per_part)
        enc.append(gather_encode(acc, fmt, dtype))
    slots = [gather_decode(e[0], fmt, perm.slots_per_part) for e in enc]
    vals = [e[1] for e in enc]
    res = densify(slots, vals, perm, dtype).reshape(shape)
    return [res.clone() for _ in range(P)]


# --------------------------------------------------------------------------- torch.distributed driver


def _all_to_all_v(chunks: list[torch.Tensor], group) -> list[torch.Tensor]:
    """Variable-size all-to-all built on ``all_to_all_single`` (works on gloo and NCCL)."""
    P = dist.get_world_size(group)
    dev = chunks[0].device
    send_counts = torch.tensor([c.numel() for c in chunks], dtype=torch.int64, device=dev)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    rc = recv_counts.tolist()
    send = torch.cat(chunks) if P > 1 else chunks[0]
    recv = torch.empty(sum(rc), dtype=send.dtype, device=dev)
    dist.all_to_all_single(recv, send, output_split_sizes=rc,
                           input_split_sizes=send_counts.tolist(), group=group)
    return list(torch.split(recv, rc))


def _all_gather_v(t: torch.Tensor, group) -> list[torch.Tensor]:
    """Variable-size all-gather: length exchange, pad to the maximum, gather, trim."""
    P = dist.get_world_size(group)
    n = torch.tensor([t.numel()], dtype=torch.int64, device=t.device)
    sizes = torch.empty(P, dtype=torch.int64, device=t.device)
    dist.all_gather_into_tensor(sizes, n, group=group)
    sizes = sizes.tolist()
    mx = max(max(sizes), 1)
    padded = torch.zeros(mx, dtype=t.dtype, device=t.device)
    padded[: t.numel()] = t
    out = torch.empty(P * mx, dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, padded, group=group)
    return [out[i * mx: i * mx + sizes[i]] for i in range(P)]


def dist_sparse_allreduce(tensor: torch.Tensor, group=None, method: int = 3, block: int = 64) -> torch.Tensor:
    """One rank's view of the sparse all-reduce over ``torch.distributed``; returns the dense SUM."""
    P = dist.get_world_size(group)
    flat = tensor.reshape(-1)
    N = flat.numel()
    if P == 1:
        return tensor.clone()
    if method == 1:
        idx = torch.nonzero(flat, as_tuple=True)[0]
        all_idx = _all_gather_v(idx, group)
        all_val = _all_gather_v(flat[idx], group)
        acc = torch.zeros(N, dtype=torch.float32, device=flat.device)
        for i, v in zip(all_idx, all_val):
            acc.index_add_(0, i, v.to(torch.float32))
        return acc.to(tensor.dtype).reshape(tensor.shape)
    perm = BlockPermutation.make(N, P, block)
    slots, vals, _ = partition(flat, perm)
    rslots = _all_to_all_v(slots, group)
    rvals = _all_to_all_v(vals, group)
    acc = owner_reduce(rslots, rvals, perm.slots_per_part)
    fmt = "bitmap" if method == 3 else "coo"
    payload, v = gather_encode(acc, fmt, tensor.dtype)
    all_payload = _all_gather_v(payload, group)
    all_vals = _all_gather_v(v, group)
    all_slots = [gather_decode(p, fmt, perm.slots_per_part) for p in all_payload]
    return densify(all_slots, all_vals, perm, tensor.dtype).reshape(tensor.shape)
