"""Row-granule sparse all-reduce of embedding gradients (CUDA engine + pure-PyTorch oracle).

Input per rank: ``rows`` (unique int32 row ids), ``count`` (device int32[1]) and ``vals[*, d]``.
Output: the element-wise SUM over ranks of the implied sparse [V, d] matrices, added (scaled) into a
dense gradient on every rank.  ``RowSparseAllReduce`` is the one-process-per-GPU engine (P2P stores
over NVLink, bounded waits, no NCCL and no host sync); ``VirtualRowSparseAllReduce`` runs all ranks
on one GPU phase by phase for tests.
"""
from __future__ import annotations

import ctypes
import math

import torch

from .. import _native
from ..runtime.symmetric import LocalSymmetric, SymmetricRegion, make_symmetric
from .engine import MAX_RANKS, _Perm, _up, perm_struct
from .hashing import BlockPermutation


class _RowCtx(ctypes.Structure):
    _fields_ = [
        ("rank", ctypes.c_int32), ("nranks", ctypes.c_int32), ("epoch", ctypes.c_uint32), ("d", ctypes.c_uint32),
        ("wait_ns", ctypes.c_uint64), ("sym", ctypes.c_void_p * MAX_RANKS),
        ("off_rec_mail", ctypes.c_uint64), ("off_g_mail", ctypes.c_uint64), ("off_rec_slot", ctypes.c_uint64),
        ("off_rec_val", ctypes.c_uint64), ("off_g_row", ctypes.c_uint64), ("off_g_val", ctypes.c_uint64),
        ("cap_rec", ctypes.c_uint32), ("cap_g", ctypes.c_uint32), ("nslots", ctypes.c_uint32), ("nwords", ctypes.c_uint32),
        ("acc", ctypes.c_void_p), ("bitmap", ctypes.c_void_p), ("list", ctypes.c_void_p), ("cursors", ctypes.c_void_p),
        ("status", ctypes.c_void_p), ("vocab", ctypes.c_uint32), ("pad", ctypes.c_uint32),
        ("epoch_dev", ctypes.c_void_p), ("perm", _Perm),
    ]


class RowPlan:
    """Sizes for (vocab, d, P): ``max_rows`` is the most rows one rank can contribute per step."""

    def __init__(self, vocab: int, d: int, nranks: int, max_rows: int, elem_size: int = 2, slack: float = 2.0):
        assert d % 8 == 0
        self.vocab, self.d, self.nranks, self.max_rows, self.elem_size = vocab, d, nranks, max_rows, elem_size
        self.perm = BlockPermutation.make(vocab, nranks, 1)
        S = self.perm.slots_per_part
        self.nslots, self.nwords = S, (S + 31) // 32
        self.cap_rec = _up(min(max_rows, math.ceil(max_rows / nranks * slack) + 64), 8)
        self.cap_g = _up(min(S, self.cap_rec * nranks), 8)
        off = 0
        self.off_rec_mail = off; off += 256
        self.off_g_mail = off; off += 256
        self.off_rec_slot = off; off += _up(nranks * self.cap_rec * 4, 256)
        self.off_rec_val = off; off += _up(nranks * self.cap_rec * d * elem_size, 256)
        self.off_g_row = off; off += _up(nranks * self.cap_g * 4, 256)
        self.off_g_val = off; off += _up(nranks * self.cap_g * d * elem_size, 256)
        self.sym_bytes = off


class RowRank:
    def __init__(self, plan: RowPlan, region: SymmetricRegion, wait_ms: float = 2000.0):
        self.plan, self.region, self.lib = plan, region, _native.lib()
        assert self.lib.zen_row_ctx_size() == ctypes.sizeof(_RowCtx), "row ctx layout mismatch"
        dev = torch.device(f"cuda:{torch.cuda.current_device()}")
        self.acc = torch.zeros(plan.nslots, plan.d, dtype=torch.float32, device=dev)
        self.bitmap = torch.zeros(plan.nwords, dtype=torch.int32, device=dev)
        self.list = torch.zeros(plan.nslots, dtype=torch.int32, device=dev)
        self.cursors = torch.zeros(MAX_RANKS + 4, dtype=torch.int32, device=dev)
        self.status_t = torch.zeros(1, dtype=torch.int32, device=dev)
        c = _RowCtx()
        c.rank, c.nranks, c.d, c.wait_ns = region.rank, region.nranks, plan.d, int(wait_ms * 1e6)
        for r in range(region.nranks):
            c.sym[r] = region.ptrs[r]
        for name in ("off_rec_mail", "off_g_mail", "off_rec_slot", "off_rec_val", "off_g_row", "off_g_val",
                     "cap_rec", "cap_g", "nslots", "nwords", "vocab"):
            setattr(c, name, getattr(plan, name))
        c.acc, c.bitmap, c.list = self.acc.data_ptr(), self.bitmap.data_ptr(), self.list.data_ptr()
        c.cursors, c.status = self.cursors.data_ptr(), self.status_t.data_ptr()
        c.perm = perm_struct(plan.perm)
        self.ctx = c

    def _p(self, epoch):
        self.ctx.epoch = epoch
        return ctypes.byref(self.ctx)

    def push(self, rows, count, vals, epoch):
        assert vals.is_contiguous() and vals.shape[1] == self.plan.d and vals.element_size() == self.plan.elem_size
        _native.check(self.lib.zen_row_push(self._p(epoch), _native.ptr(rows), _native.ptr(count), _native.ptr(vals),
                                            min(rows.numel(), vals.shape[0]), _native.DTYPE_CODE[vals.dtype],
                                            _native.stream_ptr()), "zen_row_push")

    def reduce(self, dtype, epoch, deterministic=False):
        _native.check(self.lib.zen_row_reduce(self._p(epoch), _native.DTYPE_CODE[dtype], int(deterministic),
                                              _native.stream_ptr()), "zen_row_reduce")

    def gather_push(self, dtype, epoch):
        _native.check(self.lib.zen_row_gather_push(self._p(epoch), _native.DTYPE_CODE[dtype], _native.stream_ptr()),
                      "zen_row_gather_push")

    def apply(self, grad, epoch, scale=1.0, overwrite=False):
        assert grad.is_contiguous() and grad.shape == (self.plan.vocab, self.plan.d)
        _native.check(self.lib.zen_row_apply(self._p(epoch), _native.ptr(grad), ctypes.c_float(scale), int(overwrite),
                                             _native.DTYPE_CODE[grad.dtype], _native.stream_ptr()), "zen_row_apply")

    def read_status(self, clear=True) -> int:
        v = int(self.status_t.item())
        if v and clear:
            self.status_t.zero_()
        return v


class RowSparseAllReduce:
    """One process per GPU.  ``__call__(rows, count, vals, grad)`` adds ``scale * sum_over_ranks`` into ``grad``."""

    def __init__(self, vocab, d, max_rows, group=None, dtype=torch.bfloat16, deterministic=False, wait_ms=2000.0,
                 backend=None):
        import torch.distributed as dist

        P = dist.get_world_size(group)
        self.plan = RowPlan(vocab, d, P, max_rows, torch.empty(0, dtype=dtype).element_size())
        self.region = make_symmetric(self.plan.sym_bytes, group, backend)
        self.state = RowRank(self.plan, self.region, wait_ms)
        self.deterministic, self.epoch = deterministic, 0
        self._epoch_dev = None

    def enable_device_epoch(self):
        """Keep the call counter on the device (bumped by a one-thread kernel at the start of each call), so that a
        captured sequence of calls stays in step with the peers when the graph is replayed."""
        dev = self.state.acc.device
        self._epoch_dev = torch.full((1,), self.epoch, dtype=torch.int32, device=dev)
        self.state.ctx.epoch_dev = self._epoch_dev.data_ptr()

    def start(self, rows, count, vals):
        """First three stages (push to the owners, owner reduce, push of the reduced rows to every rank): needs only this
        rank's rows, so it can run on a side stream while the dense gradient is still being reduced."""
        self.epoch += 1
        if self._epoch_dev is not None:
            _native.check(self.state.lib.zen_row_epoch_bump(_native.ptr(self._epoch_dev), _native.stream_ptr()),
                          "zen_row_epoch_bump")
        e, s = self.epoch, self.state
        s.push(rows, count, vals, e)
        s.reduce(vals.dtype, e, self.deterministic)
        s.gather_push(vals.dtype, e)

    def finish(self, grad, scale=1.0, overwrite=False):
        """Last stage: add (or write) the gathered rows into the dense gradient."""
        self.state.apply(grad, self.epoch, scale, overwrite)
        return grad

    def __call__(self, rows, count, vals, grad, scale=1.0, overwrite=False):
        self.start(rows, count, vals)
        return self.finish(grad, scale, overwrite)

    def check(self) -> int:
        return self.state.read_status()

    def close(self):
        self.region.close()


class VirtualRowSparseAllReduce:
    def __init__(self, vocab, d, max_rows, nranks, dtype=torch.bfloat16, deterministic=True):
        self.plan = RowPlan(vocab, d, nranks, max_rows, torch.empty(0, dtype=dtype).element_size())
        self.sym = LocalSymmetric(nranks, self.plan.sym_bytes)
        self.ranks = [RowRank(self.plan, self.sym.for_rank(r), wait_ms=50.0) for r in range(nranks)]
        self.deterministic, self.epoch = deterministic, 0

    def __call__(self, rows_l, count_l, vals_l, grads, scale=1.0, overwrite=False):
        self.epoch += 1
        e = self.epoch
        for r, rows, cnt, vals in zip(self.ranks, rows_l, count_l, vals_l):
            r.push(rows, cnt, vals, e)
        for r, vals in zip(self.ranks, vals_l):
            r.reduce(vals.dtype, e, self.deterministic)
        for r, vals in zip(self.ranks, vals_l):
            r.gather_push(vals.dtype, e)
        for r, g in zip(self.ranks, grads):
            r.apply(g, e, scale, overwrite)
        return grads

    def status(self):
        return [r.read_status() for r in self.ranks]


def rows_oracle(rows_l, count_l, vals_l, vocab, d, scale=1.0):
    """Dense fp32 [vocab, d] sum of every rank's sparse rows (rank order), times ``scale``."""
    acc = torch.zeros(vocab, d, dtype=torch.float32)
    for rows, cnt, vals in zip(rows_l, count_l, vals_l):
        n = int(cnt.item())
        acc.index_add_(0, rows[:n].cpu().long(), vals[:n].float().cpu())
    return acc * scale


def dist_rows_allreduce(rows, count, vals, grad, group=None, scale=1.0):
    """Library path (gloo / NCCL): all-gather of (rows, vals) padded to the maximum count, then index_add."""
    import torch.distributed as dist

    P = dist.get_world_size(group)
    n = int(count.item())
    cnts = torch.zeros(P, dtype=torch.int64, device=rows.device)
    dist.all_gather_into_tensor(cnts, torch.tensor([n], dtype=torch.int64, device=rows.device), group=group)
    mx = max(int(cnts.max()), 1)
    d = vals.shape[1]
    r_pad = torch.zeros(mx, dtype=torch.int32, device=rows.device); r_pad[:n] = rows[:n]
    v_pad = torch.zeros(mx, d, dtype=vals.dtype, device=rows.device); v_pad[:n] = vals[:n]
    all_r = torch.empty(P * mx, dtype=torch.int32, device=rows.device)
    all_v = torch.empty(P * mx, d, dtype=vals.dtype, device=rows.device)
    dist.all_gather_into_tensor(all_r, r_pad, group=group)
    dist.all_gather_into_tensor(all_v, v_pad, group=group)
    acc = torch.zeros(grad.shape, dtype=torch.float32, device=grad.device)
    for p in range(P):
        k = int(cnts[p])
        acc.index_add_(0, all_r[p * mx: p * mx + k].long(), all_v[p * mx: p * mx + k].float())
    grad.add_((acc * scale).to(grad.dtype))
    return grad
