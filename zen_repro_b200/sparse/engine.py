"""CUDA sparse all-reduce engine: plans buffers, owns the per-rank state, launches the kernels.

``SparseAllReduce``         one process per GPU; peers are reached through a
                            symmetric region (P2P stores over NVLink).  No NCCL
                            call on the data path and no host synchronisation.
``VirtualSparseAllReduce``  all ``P`` ranks on one GPU, run phase by phase (a
                            consumer phase only starts after every producer of
                            the previous phase has finished, so nothing ever
                            spins).  Used by single-GPU tests and benchmarks.

Method numbers follow the reference (comm.py:101-146): 1 sparse all-gather,
2 balanced exchange + COO gather, 3 balanced exchange + bitmap gather; plus
``"auto"`` which lets every owner choose COO or bitmap from its union count.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field

import torch

from .. import _native
from ..runtime.symmetric import LocalSymmetric, SymmetricRegion, make_symmetric
from .hashing import BlockPermutation

MAX_RANKS = 8
ST_REC_OVERFLOW, ST_GATHER_OVERFLOW, ST_TIMEOUT, ST_PEER_OVERFLOW, ST_BAD_ARG = 1, 2, 4, 8, 16
FMT_AUTO, FMT_COO, FMT_BITMAP = 0, 1, 2


class _Perm(ctypes.Structure):
    _fields_ = [("block", ctypes.c_uint32), ("nblocks", ctypes.c_uint32), ("sb", ctypes.c_uint32),
                ("mask", ctypes.c_uint32), ("mult", ctypes.c_uint32), ("mult_inv", ctypes.c_uint32),
                ("add", ctypes.c_uint32), ("lg", ctypes.c_uint32)]


class _Ctx(ctypes.Structure):
    _fields_ = [
        ("rank", ctypes.c_int32), ("nranks", ctypes.c_int32), ("epoch", ctypes.c_uint32),
        ("fmt_mode", ctypes.c_uint32), ("wait_ns", ctypes.c_uint64),
        ("sym", ctypes.c_void_p * MAX_RANKS),
        ("off_rec_mail", ctypes.c_uint64), ("off_g_mail", ctypes.c_uint64), ("off_rec", ctypes.c_uint64),
        ("off_g_idx", ctypes.c_uint64), ("off_g_off", ctypes.c_uint64), ("off_g_val", ctypes.c_uint64),
        ("cap_rec", ctypes.c_uint32), ("cap_g", ctypes.c_uint32), ("g_idx_words", ctypes.c_uint32),
        ("nchunks", ctypes.c_uint32),
        ("acc", ctypes.c_void_p), ("bitmap", ctypes.c_void_p), ("chunk_off", ctypes.c_void_p),
        ("cursors", ctypes.c_void_p), ("status", ctypes.c_void_p),
        ("numel", ctypes.c_uint64), ("nslots", ctypes.c_uint32), ("nwords", ctypes.c_uint32),
        ("perm", _Perm),
    ]


def perm_struct(perm: BlockPermutation) -> _Perm:
    return _Perm(perm.block, perm.nblocks, perm.blocks_per_part, perm.mask, perm.mult, perm.mult_inv, perm.add,
                 perm.block.bit_length() - 1)


def _up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


@dataclass
class SparsePlan:
    """Sizes and symmetric-region layout for one (numel, P) pair."""

    numel: int
    nranks: int
    block: int = 64
    max_density: float = 0.12      # largest per-rank nonzero fraction served without fallback
    slack: float = 1.3
    method1: bool = False          # size record slots for a full sparse all-gather
    forced_coo: bool = False       # size the index payload for COO at any union count
    perm: BlockPermutation = field(init=False)

    def __post_init__(self):
        if not (1 <= self.nranks <= MAX_RANKS):
            raise ValueError(f"nranks must be in [1, {MAX_RANKS}]")
        if self.block < 64 or self.block & (self.block - 1):
            raise ValueError("element-granule block must be a power of two >= 64")
        if self.numel >= 2 ** 32 - 4096:
            raise ValueError("numel must fit 32-bit indices")
        self.perm = BlockPermutation.make(self.numel, self.nranks, self.block)
        P, S = self.nranks, self.perm.slots_per_part
        nnz = min(self.numel, math.ceil(self.numel * self.max_density))
        per_pair = nnz if self.method1 else math.ceil(nnz / P * self.slack)
        self.cap_rec = _up(min(per_pair + 1024, self.numel + 64), 8)
        union = min(S, math.ceil(S * min(1.0, self.max_density * P) * self.slack))
        self.cap_g = _up(max(union, 64), 8)
        self.nwords = (S + 31) // 32
        self.nchunks = (S + 1023) // 1024
        self.g_idx_words = _up(max(self.nwords, self.cap_g if self.forced_coo else 0), 4)
        off = 0
        self.off_rec_mail = off; off += _up(16 * MAX_RANKS, 256)
        self.off_g_mail = off; off += _up(16 * MAX_RANKS, 256)
        self.off_rec = off; off += _up(P * self.cap_rec * 8, 256)
        self.off_g_idx = off; off += _up(P * self.g_idx_words * 4, 256)
        self.off_g_off = off; off += _up(P * (self.nchunks + 1) * 4, 256)
        self.off_g_val = off; off += _up(P * self.cap_g * 4, 256)
        self.sym_bytes = off

    @property
    def nslots(self) -> int:
        return self.perm.slots_per_part


class SparseRank:
    """One rank's buffers and kernel launches."""

    def __init__(self, plan: SparsePlan, region: SymmetricRegion, wait_ms: float = 2000.0):
        self.plan, self.region = plan, region
        self.lib = _native.lib()
        assert self.lib.zen_sparse_ctx_size() == ctypes.sizeof(_Ctx), "ctx layout mismatch"
        dev = torch.device(f"cuda:{torch.cuda.current_device()}")
        self.acc = torch.zeros(plan.nslots, dtype=torch.float32, device=dev)
        self.bitmap = torch.zeros(plan.nwords, dtype=torch.int32, device=dev)
        self.chunk_off = torch.zeros(plan.nchunks + 1, dtype=torch.int32, device=dev)
        self.cursors = torch.zeros(MAX_RANKS + 2, dtype=torch.int32, device=dev)
        self.status_t = torch.zeros(1, dtype=torch.int32, device=dev)
        c = _Ctx()
        c.rank, c.nranks = region.rank, region.nranks
        c.wait_ns = int(wait_ms * 1e6)
        for r in range(region.nranks):
            c.sym[r] = region.ptrs[r]
        for name in ("off_rec_mail", "off_g_mail", "off_rec", "off_g_idx", "off_g_off", "off_g_val",
                     "cap_rec", "cap_g", "g_idx_words", "nchunks", "nwords"):
            setattr(c, name, getattr(plan, name))
        c.acc, c.bitmap = self.acc.data_ptr(), self.bitmap.data_ptr()
        c.chunk_off, c.cursors, c.status = self.chunk_off.data_ptr(), self.cursors.data_ptr(), self.status_t.data_ptr()
        c.numel, c.nslots = plan.numel, plan.nslots
        c.perm = perm_struct(plan.perm)
        self.ctx = c

    def _prep(self, epoch: int, fmt: int = FMT_AUTO):
        self.ctx.epoch = epoch
        self.ctx.fmt_mode = fmt
        return ctypes.byref(self.ctx)

    def partition_push(self, x: torch.Tensor, epoch: int, thr: torch.Tensor | None = None, broadcast: bool = False):
        assert x.is_cuda and x.is_contiguous() and x.numel() == self.plan.numel
        rc = self.lib.zen_partition_push(self._prep(epoch), _native.ptr(x), _native.ptr(thr),
                                         _native.DTYPE_CODE[x.dtype], int(broadcast), _native.stream_ptr())
        _native.check(rc, "zen_partition_push")

    def owner_reduce(self, epoch: int, dtype: torch.dtype, deterministic: bool = False):
        rc = self.lib.zen_owner_reduce(self._prep(epoch), _native.DTYPE_CODE[dtype], int(deterministic),
                                       _native.stream_ptr())
        _native.check(rc, "zen_owner_reduce")

    def gather_push(self, epoch: int, dtype: torch.dtype, fmt: int = FMT_AUTO):
        rc = self.lib.zen_gather_push(self._prep(epoch, fmt), _native.DTYPE_CODE[dtype], _native.stream_ptr())
        _native.check(rc, "zen_gather_push")

    def densify(self, out: torch.Tensor, epoch: int, fmt: int = FMT_AUTO):
        assert out.is_contiguous() and out.numel() == self.plan.numel and out.data_ptr() % 16 == 0
        rc = self.lib.zen_densify(self._prep(epoch, fmt), _native.ptr(out), _native.DTYPE_CODE[out.dtype],
                                  _native.stream_ptr())
        _native.check(rc, "zen_densify")

    def scatter_sources(self, out: torch.Tensor, epoch: int):
        rc = self.lib.zen_scatter_sources(self._prep(epoch), _native.ptr(out), _native.DTYPE_CODE[out.dtype],
                                          _native.stream_ptr())
        _native.check(rc, "zen_scatter_sources")

    def read_status(self, clear: bool = True) -> int:
        """Host read of the status word (synchronises the current stream)."""
        v = int(self.status_t.item())
        if clear and v:
            self.status_t.zero_()
        return v


def _fmt_for(method) -> int:
    return {2: FMT_COO, 3: FMT_BITMAP, "auto": FMT_AUTO, 0: FMT_AUTO}.get(method, FMT_AUTO)


def status_message(st: int) -> str:
    names = [(ST_REC_OVERFLOW, "record slot overflow"), (ST_GATHER_OVERFLOW, "gather payload overflow"),
             (ST_TIMEOUT, "peer wait timed out"), (ST_PEER_OVERFLOW, "peer reported overflow"),
             (ST_BAD_ARG, "out-of-range slot")]
    return ", ".join(n for b, n in names if st & b) or "ok"


class SparseAllReduce:
    """Sparse all-reduce (SUM) of a flat bucket across a process group, one process per GPU.

    ``__call__`` enqueues four to six kernels on the current stream and returns
    the dense result without synchronising.  ``check()`` reads the status word;
    on overflow every rank sees the same status (overflow bits travel in the
    mails), so the caller can fall back to a dense all-reduce collectively.
    """

    def __init__(self, numel: int, group=None, *, block: int = 64, max_density: float = 0.12,
                 methods=(3,), deterministic: bool = False, wait_ms: float = 2000.0, backend: str | None = None):
        import torch.distributed as dist

        self.group = group
        P = dist.get_world_size(group)
        self.plan = SparsePlan(numel, P, block, max_density, method1=1 in methods, forced_coo=2 in methods)
        self.region = make_symmetric(self.plan.sym_bytes, group, backend)
        self.rank_state = SparseRank(self.plan, self.region, wait_ms)
        self.deterministic = deterministic
        self.epoch = 0

    def __call__(self, x: torch.Tensor, method=3, out: torch.Tensor | None = None,
                 threshold: torch.Tensor | None = None) -> torch.Tensor:
        flat = x.reshape(-1)
        if out is None:
            out = torch.empty_like(flat)
        self.epoch += 1
        e, rs = self.epoch, self.rank_state
        if method == 1:
            rs.partition_push(flat, e, threshold, broadcast=True)
            rs.scatter_sources(out.reshape(-1), e)
        else:
            fmt = _fmt_for(method)
            rs.partition_push(flat, e, threshold)
            rs.owner_reduce(e, flat.dtype, self.deterministic)
            rs.gather_push(e, flat.dtype, fmt)
            rs.densify(out.reshape(-1), e, fmt)
        return out.reshape(x.shape)

    def check(self) -> int:
        return self.rank_state.read_status()

    def close(self):
        self.region.close()


class VirtualSparseAllReduce:
    """All ``P`` ranks on one device, executed phase by phase on the current stream."""

    def __init__(self, numel: int, nranks: int, *, block: int = 64, max_density: float = 0.12,
                 methods=(3,), deterministic: bool = False):
        self.plan = SparsePlan(numel, nranks, block, max_density, method1=1 in methods, forced_coo=2 in methods)
        self.sym = LocalSymmetric(nranks, self.plan.sym_bytes)
        self.ranks = [SparseRank(self.plan, self.sym.for_rank(r), wait_ms=50.0) for r in range(nranks)]
        self.deterministic = deterministic
        self.epoch = 0

    def __call__(self, inputs, method=3, threshold: torch.Tensor | None = None):
        assert len(inputs) == self.plan.nranks
        self.epoch += 1
        e = self.epoch
        flats = [t.reshape(-1) for t in inputs]
        outs = [torch.empty_like(f) for f in flats]
        if method == 1:
            for r, f in zip(self.ranks, flats):
                r.partition_push(f, e, threshold, broadcast=True)
            for r, o in zip(self.ranks, outs):
                r.scatter_sources(o, e)
        else:
            fmt = _fmt_for(method)
            for r, f in zip(self.ranks, flats):
                r.partition_push(f, e, threshold)
            for r, f in zip(self.ranks, flats):
                r.owner_reduce(e, f.dtype, self.deterministic)
            for r, f in zip(self.ranks, flats):
                r.gather_push(e, f.dtype, fmt)
            for r, o in zip(self.ranks, outs):
                r.densify(o, e, fmt)
        return [o.reshape(t.shape) for o, t in zip(outs, inputs)]

    def status(self) -> list[int]:
        return [r.read_status() for r in self.ranks]
