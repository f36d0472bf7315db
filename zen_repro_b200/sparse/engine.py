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
from ..utils import trace
from ..runtime.symmetric import LocalSymmetric, SymmetricRegion, make_symmetric
from .hashing import BlockPermutation

MAX_RANKS = 8
ST_REC_OVERFLOW, ST_GATHER_OVERFLOW, ST_TIMEOUT, ST_PEER_OVERFLOW, ST_BAD_ARG = 1, 2, 4, 8, 16
FMT_AUTO, FMT_COO, FMT_BITMAP = 0, 1, 2
CANARY_BYTES, CANARY_WORD = 256, 0x5AFEC0DE


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
        ("epoch_dev", ctypes.c_void_p), ("mc", ctypes.c_void_p),
        ("k1_density_ppm", ctypes.c_uint32), ("pad0", ctypes.c_uint32),
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
        self.nwords = (S + 31) // 32
        self.nchunks = (S + 1023) // 1024
        ngroups = self.nchunks              # one run per 1024-slot chunk
        # the gather payload is filled in runs that start on 8-value boundaries: up to 8 padding values per run
        self.cap_g = _up(max(union, 64) + 8 * ngroups, 8)
        # bitmap words, or a COO list: the whole payload when format 2 is forced, else as many entries as the
        # automatic choice can pick COO for (at most one touched slot in 32) plus the padding between runs
        self.g_idx_words = _up(max(self.nwords, self.cap_g) if self.forced_coo else self.nwords + 8 * ngroups + 64, 4)
        # sub-regions of the symmetric region, each followed by a guard of CANARY_BYTES that nothing may write
        off, self.canaries = 0, []

        def take(nbytes):
            nonlocal off
            at = off
            off += _up(nbytes, 256)
            self.canaries.append(off)
            off += CANARY_BYTES
            return at

        self.off_rec_mail = take(2 * 16 * MAX_RANKS)                      # two parities
        self.off_g_mail = take(16 * MAX_RANKS)
        self.off_rec = take(2 * P * self.cap_rec * 8)                     # two parities
        self.off_g_idx = take(P * self.g_idx_words * 4)
        self.off_g_off = take(P * (self.nchunks + 1) * 4)
        self.off_g_val = take(P * self.cap_g * 4)
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
        self.cursors = torch.zeros(MAX_RANKS + 4, dtype=torch.int32, device=dev)
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
        c.k1_density_ppm = max(1, min(1_000_000, int(plan.max_density * 1e6)))
        c.mc = getattr(region, "multicast_ptr", 0) if getattr(region, "use_multicast", False) else 0
        self.ctx = c
        self.epoch_dev = None
        for at in plan.canaries:                                      # guard words after every sub-region of OUR region
            region.view(region.rank, at, CANARY_BYTES, torch.int32).fill_(CANARY_WORD)

    def damaged_canaries(self) -> list[int]:
        """Offsets of guard zones in this rank's region whose pattern was overwritten (by a peer's or an own store that
        ran past its sub-region).  Synchronises; for tests and health checks."""
        bad = []
        for at in self.plan.canaries:
            if not bool((self.region.view(self.region.rank, at, CANARY_BYTES, torch.int32) == CANARY_WORD).all()):
                bad.append(at)
        return bad

    def enable_device_epoch(self, start: int = 0):
        """Keep the call counter on the device: every kernel reads it there and ``allreduce`` bumps it first, so a
        captured sequence of calls stays in step with the peers when the graph is replayed."""
        self.epoch_dev = torch.full((1,), start, dtype=torch.int32, device=self.acc.device)
        self.ctx.epoch_dev = self.epoch_dev.data_ptr()

    def allreduce(self, x: torch.Tensor, out: torch.Tensor, epoch: int, thr: torch.Tensor | None = None,
                  method1: bool = False, fmt: int = FMT_AUTO, deterministic: bool = False):
        """All kernels of one call from a single native entry."""
        assert x.is_cuda and x.is_contiguous() and x.numel() == self.plan.numel
        assert out.is_contiguous() and out.numel() == self.plan.numel and out.data_ptr() % 16 == 0
        # ``out`` may be ``x`` itself: this rank's scan of ``x`` has finished (stream order) before anything is written
        rc = self.lib.zen_sparse_allreduce(self._prep(epoch, fmt), _native.ptr(x), _native.ptr(thr), _native.ptr(out),
                                           _native.DTYPE_CODE[x.dtype], int(method1), int(deterministic),
                                           _native.stream_ptr())
        _native.check(rc, "zen_sparse_allreduce")

    def metrics(self, epoch: int) -> dict:
        """What the mails of call ``epoch`` say (synchronises): records this owner received from every source, touched
        slots per owner as gathered here (padding between runs included), index format per owner."""
        P = self.region.nranks
        rm = self.region.view(self.region.rank, self.plan.off_rec_mail, 2 * 16 * MAX_RANKS, torch.int32).view(2, MAX_RANKS, 4)
        gm = self.region.view(self.region.rank, self.plan.off_g_mail, 16 * MAX_RANKS, torch.int32).view(MAX_RANKS, 4)
        rm, gm = rm[epoch & 1, :P].cpu(), gm[:P].cpu()
        ok_r = [int(e) == epoch for e in rm[:, 3]]
        ok_g = [int(e) == epoch for e in gm[:, 3]]
        return {"recv_records": [int(c) if ok else None for c, ok in zip(rm[:, 0], ok_r)],
                "gathered": [int(c) if ok else None for c, ok in zip(gm[:, 0], ok_g)],
                "format": [{FMT_COO: "coo", FMT_BITMAP: "bitmap"}.get((int(i) >> 8) & 0xff, "none") for i in gm[:, 1]]}

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
                 methods=(3,), deterministic: bool = False, wait_ms: float = 2000.0, backend: str | None = None,
                 transport: str = "p2p"):
        """``transport``: "p2p" pushes the gathered payload to every peer with its own stores; "nvls" writes it once
        to the multicast alias of the region and lets the NVSwitch replicate it (needs the torch symmetric-memory
        backend and a fabric that offers multicast; falls back to "p2p" otherwise)."""
        import torch.distributed as dist

        self.group = group
        P = dist.get_world_size(group)
        self.plan = SparsePlan(numel, P, block, max_density, method1=1 in methods, forced_coo=2 in methods)
        self.transport = transport
        if transport == "nvls":
            self.region = make_symmetric(self.plan.sym_bytes, group, "torch")
            self.region.use_multicast = bool(getattr(self.region, "multicast_ptr", 0))
            if not self.region.use_multicast:
                self.transport = "p2p"
        else:
            self.region = make_symmetric(self.plan.sym_bytes, group, backend)
        self.rank_state = SparseRank(self.plan, self.region, wait_ms)
        self.deterministic = deterministic
        self.epoch = 0
        self.calls = 0
        self.timer = None              # a utils.trace.StageTimer: per-stage CUDA-event times (stage-by-stage launches)

    def metrics(self) -> dict:
        """Counters of the last call (synchronises the device): density of what this owner received, touched slots
        over all owners, bytes this rank pushed over the links, index formats."""
        torch.cuda.synchronize()
        P, plan = self.plan.nranks, self.plan
        m = self.rank_state.metrics(self.epoch)
        recv = [c for c in m["recv_records"] if c is not None]
        gath = [c for c in m["gathered"] if c is not None]
        es = 4
        out = {"numel": plan.numel, "ranks": P, "owner_recv_records": sum(recv), "owner_recv_density": sum(recv) / max(1, plan.nslots * P),
               "union_slots": sum(gath), "union_density": sum(gath) / max(1, plan.numel), "format": m["format"],
               "gather_bytes_pushed": (P - 1) * ((gath[self.region.rank] if len(gath) == P else 0) * es + plan.nwords * 4),
               "calls": self.calls}
        return out

    def __call__(self, x: torch.Tensor, method=3, out: torch.Tensor | None = None,
                 threshold: torch.Tensor | None = None) -> torch.Tensor:
        flat = x.reshape(-1)
        if out is None:
            out = torch.empty_like(flat)
        self.epoch += 1
        e, rs, fmt = self.epoch, self.rank_state, _fmt_for(method)
        self.calls += 1
        if not trace.tracing_enabled() and self.timer is None:
            rs.allreduce(flat, out.reshape(-1), e, threshold, method1=(method == 1), fmt=fmt, deterministic=self.deterministic)
        else:
            # stage by stage, under the range names that the reference gives the corresponding steps (comm.py:104-146,
            # tensor_load_balance.py:25-44); with ``timer`` set every stage is also bracketed by CUDA events
            stage = self.timer.stage if self.timer is not None else trace.trace_range
            if rs.epoch_dev is not None:
                _native.check(rs.lib.zen_sparse_epoch_bump(_native.ptr(rs.epoch_dev), _native.stream_ptr()), "zen_sparse_epoch_bump")
            if method == 1:
                with stage("encode_sparse_tensor"):
                    rs.partition_push(flat, e, threshold, broadcast=True)
                with stage("decode_sparse_tensors"):
                    rs.scatter_sources(out.reshape(-1), e)
            else:
                with stage("load_balance"):                    # + "alltoallv indices" / "alltoallv values": pushed in the scan
                    rs.partition_push(flat, e, threshold)
                with stage("decode_sparse_tensors"):           # owner-side scatter-add
                    rs.owner_reduce(e, flat.dtype, self.deterministic)
                with stage("encode_bitmap" if fmt == FMT_BITMAP else "encode_sparse_tensor"):   # + "allgatherv"
                    rs.gather_push(e, flat.dtype, fmt)
                with stage("decode_bitmap" if fmt == FMT_BITMAP else "decode_sparse_tensors"):
                    rs.densify(out.reshape(-1), e, fmt)
        return out.reshape(x.shape)

    def enable_device_epoch(self):
        self.rank_state.enable_device_epoch(self.epoch)

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
