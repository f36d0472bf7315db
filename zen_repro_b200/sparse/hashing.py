"""Partition functions for the sparse all-reduce.

Two partitioners are provided.

``BlockPermutation`` (default).  An invertible permutation of *blocks* of ``G``
consecutive elements, cheap enough to evaluate per block inside the scan kernel
(32-bit multiply-add, no division by a runtime modulus).  With ``nb' = P * Sb``
padded blocks and ``2**k`` the next power of two >= ``nb'``,

    f(y)     = (a * y + c) mod 2**k           (a odd, so f is a bijection of [0, 2**k))
    pi(b)    = f applied to b until the value is < nb'       (cycle walking)
    owner(i) = pi(i // G) // Sb
    slot(i)  = (pi(i // G) % Sb) * G + i % G
    i        = pi^-1(owner * Sb + slot // G) * G + slot % G

``a`` is the odd integer nearest ``2**k / golden_ratio`` and the owner is taken
from the HIGH bits of ``pi`` (Fibonacci hashing), which spreads any contiguous
run of hot positions (the Zipf head of an embedding table) evenly over the
``P`` owners.  Cycle walking restricts the power-of-two bijection to
``[0, nb')`` and keeps it a bijection; since ``nb' > 2**(k-1)`` it needs less
than one extra step on average.  Because the map is invertible the owner can
reduce into ``S = Sb * G`` dense slots and the occupancy bitmap of those slots
*is* the index encoding of the gather phase; no per-position ownership list has
to be stored, and sizes that are not multiples of ``P`` need no special case.
The reference builds its ownership lists by hashing every position and
comparing against each rank (comm.py:52-56) and its two hash users disagree
when ``numel % P != 0`` (functions_cuda_kernel.cu:172-174 vs
tensor_load_balance.py:15-16).

``zen_poly3``.  The reference's cubic polynomial in wrapping uint32
arithmetic (functions_cuda_kernel.cu:80-93), kept for A/B checks of the
partition assignment: ``owner(i) = (h(i, seed0) % M) // (M // P)``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

GOLDEN = 0.6180339887498949

ZEN_POLY3_D = 573729859
ZEN_POLY3_A = 0xCC9E2D51
ZEN_POLY3_B = 0x1B873593
ZEN_SEEDS = (10001861, 100703, 5002639)

_MAX_WALK = 64


@dataclass(frozen=True)
class BlockPermutation:
    """Invertible block permutation; see the module docstring for the maths."""

    numel: int            # N: logical elements (or rows in row mode)
    parts: int            # P
    block: int            # G
    nblocks: int          # nb' (padded, multiple of P)
    blocks_per_part: int  # Sb
    mask: int             # 2**k - 1
    mult: int             # a (odd)
    mult_inv: int         # a^-1 mod 2**k
    add: int              # c

    @staticmethod
    def make(numel: int, parts: int, block: int = 64) -> "BlockPermutation":
        if numel <= 0 or parts <= 0 or block <= 0:
            raise ValueError("numel, parts and block must be positive")
        nb = -(-numel // block)
        sb = -(-nb // parts)
        nbp = sb * parts
        if nbp >= 2 ** 31:
            raise ValueError("too many blocks for 32-bit block ids")
        k = max(1, (nbp - 1).bit_length())
        size = 1 << k
        a = int(round(size * GOLDEN)) | 1
        ainv = pow(a, -1, size)
        c = int(round(size * (1.0 - GOLDEN) * 0.5)) & (size - 1)
        return BlockPermutation(numel, parts, block, nbp, sb, size - 1, a, ainv, c)

    @property
    def slots_per_part(self) -> int:
        return self.blocks_per_part * self.block

    @property
    def padded_numel(self) -> int:
        return self.nblocks * self.block

    # -- tensor forms (int64 in, int64 out) ---------------------------------
    def _walk(self, y: torch.Tensor, step) -> torch.Tensor:
        y = step(y)
        for _ in range(_MAX_WALK):
            out = y >= self.nblocks
            if not bool(out.any()):
                return y
            y = torch.where(out, step(y), y)
        raise RuntimeError("cycle walk did not terminate")

    def permute_block(self, blk: torch.Tensor) -> torch.Tensor:
        return self._walk(blk.to(torch.int64), lambda y: (y * self.mult + self.add) & self.mask)

    def unpermute_block(self, pb: torch.Tensor) -> torch.Tensor:
        return self._walk(pb.to(torch.int64), lambda y: ((y - self.add) & self.mask) * self.mult_inv & self.mask)

    def owner_slot(self, idx: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        idx = idx.to(torch.int64)
        pb = self.permute_block(idx // self.block)
        owner = pb // self.blocks_per_part
        slot = (pb % self.blocks_per_part) * self.block + idx % self.block
        return owner, slot

    def index_of(self, owner: int | torch.Tensor, slot: torch.Tensor) -> torch.Tensor:
        slot = slot.to(torch.int64)
        pb = owner * self.blocks_per_part + slot // self.block
        return self.unpermute_block(pb) * self.block + slot % self.block


def zen_poly3(idx: torch.Tensor, seed: int) -> torch.Tensor:
    """h(k, c) = d k^3 + a k^2 + b k + c in wrapping uint32 arithmetic (int64 tensor out)."""
    m = 0xFFFFFFFF
    k = idx.to(torch.int64) & m
    k2 = (k * k) & m
    k3 = (k2 * k) & m
    h = ((ZEN_POLY3_D * k3) & m) + ((ZEN_POLY3_A * k2) & m) + ((ZEN_POLY3_B * k) & m) + seed
    return h & m


def _rotl32(x: torch.Tensor, r: int) -> torch.Tensor:
    m = 0xFFFFFFFF
    return ((x << r) | (x >> (32 - r))) & m


def fmix32(h: torch.Tensor) -> torch.Tensor:
    """Finaliser of MurmurHash3 (functions_cuda_kernel.cu:27-36 in the reference, unused there)."""
    m = 0xFFFFFFFF
    h = h & m
    h = h ^ (h >> 16)
    h = (h * 0x85EBCA6B) & m
    h = h ^ (h >> 13)
    h = (h * 0xC2B2AE35) & m
    return h ^ (h >> 16)


def murmur3_32(idx: torch.Tensor, seed: int = 0) -> torch.Tensor:
    """MurmurHash3_x86_32 of each index taken as one little-endian 4-byte key (int64 tensor out, values < 2^32).
    The reference carries this hash as dead code next to the polynomial it actually uses
    (functions_cuda_kernel.cu:12-77); here it is an alternative integer mixer for experiments with the balancer."""
    m = 0xFFFFFFFF
    k = idx.to(torch.int64) & m
    k = (k * 0xCC9E2D51) & m
    k = _rotl32(k, 15)
    k = (k * 0x1B873593) & m
    h = torch.full_like(k, seed & m) ^ k
    h = _rotl32(h, 13)
    h = (h * 5 + 0xE6546B64) & m
    h = h ^ 4                                   # key length in bytes
    return fmix32(h)


def zen_poly3_owner(idx: torch.Tensor, table_size: int, parts: int) -> torch.Tensor:
    """Owner of ``idx`` under the reference balancer: first probe decides the partition."""
    per = table_size // parts
    return (zen_poly3(idx, ZEN_SEEDS[0]) % table_size) // per


def partition_imbalance(owner: torch.Tensor, parts: int) -> float:
    """max / mean load over partitions (1.0 is perfect)."""
    counts = torch.bincount(owner.to(torch.int64), minlength=parts).to(torch.float64)
    mean = counts.mean().item()
    return float(counts.max().item() / mean) if mean > 0 else 1.0
