"""Workspace and entry points of the GEMMs fused with a tensor-parallel collective (all-reduce, reduce-scatter of
the output rows, all-gather of the input rows).

``FusedTPWorkspace`` owns the symmetric exchange region of one TP group (two parities of partial-tile
buffers and per-tile flags per peer) and the call counter that every rank advances in lockstep.
``gemm_ar_*`` run the tcgen05 GEMM whose epilogue pushes bf16 partial tiles into the peers' regions with
P2P stores and sums the partials tile by tile behind bounded waits; they replace "GEMM, then NCCL
all-reduce" of a row-parallel forward and of a column-parallel input-gradient (the shardformer layers the
reference gets from ColossalAI, train.py:117-123).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from .. import _native
from ..runtime.symmetric import make_symmetric


class _ArCtx(ctypes.Structure):
    _fields_ = [("nranks", ctypes.c_int32), ("rank", ctypes.c_int32), ("epoch", ctypes.c_uint32),
                ("max_tiles", ctypes.c_uint32), ("wait_ns", ctypes.c_uint64), ("slot_elems", ctypes.c_uint64),
                ("recv", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8), ("status", ctypes.c_void_p),
                ("epoch_dev", ctypes.c_void_p), ("epoch_stride", ctypes.c_uint32), ("pad", ctypes.c_uint32)]


class FusedTPWorkspace:
    def __init__(self, group, max_rows: int, max_cols: int, wait_ms: float = 2000.0, backend: str | None = None):
        self.group = group
        self.P = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        lib = _native.lib()
        assert lib.zen_gemm_ar_ctx_size() == ctypes.sizeof(_ArCtx), "AR ctx layout mismatch"
        npeers = max(1, self.P - 1)
        self.slot_elems = max_rows * ((max_cols + 7) // 8 * 8)
        self.max_tiles = ((max_rows + 127) // 128) * ((max_cols + 127) // 128)
        flag_bytes = (2 * npeers * self.max_tiles * 4 + 255) // 256 * 256
        recv_bytes = 2 * npeers * self.slot_elems * 2
        self.region = make_symmetric(flag_bytes + recv_bytes, group, backend)
        self.status = torch.zeros(1, dtype=torch.int32, device=f"cuda:{torch.cuda.current_device()}")
        c = _ArCtx()
        c.nranks, c.rank, c.max_tiles, c.wait_ns, c.slot_elems = self.P, self.rank, self.max_tiles, int(wait_ms * 1e6), self.slot_elems
        for r in range(self.P):
            c.flags[r] = self.region.ptrs[r]
            c.recv[r] = self.region.ptrs[r] + flag_bytes
        c.status = self.status.data_ptr()
        self.ctx = c
        self.epoch = 0
        self.calls_in_step = 0             # calls since the last begin_step()
        self.calls_last_step = 0
        self._step_dev = None              # device step counter (CUDA-graph mode)

    def begin_step(self):
        """Mark the start of a training step.  In device-counter mode this launches the one-thread kernel that advances
        the step counter; every call of the step then carries only its index within the step by value."""
        self.calls_last_step, self.calls_in_step = self.calls_in_step, 0
        if self._step_dev is not None:
            _native.check(_native.lib().zen_sparse_epoch_bump(_native.ptr(self._step_dev), _native.stream_ptr()),
                          "zen_sparse_epoch_bump")

    def enable_device_epoch(self, calls_per_step: int) -> bool:
        """Derive the call counter from a step counter on the device (counter = step * stride + index in the step), so
        that a captured step sees fresh counter values at every replay.  The stride has the parity of the number of
        calls per step: consecutive calls then keep alternating between the two exchange buffers across the step
        boundary.  Every rank of the group must pass the same ``calls_per_step``."""
        stride = calls_per_step + 2
        self._step_dev = torch.full((1,), self.epoch // stride + 1, dtype=torch.int32, device=self.status.device)
        self.ctx.epoch_dev = self._step_dev.data_ptr()
        self.ctx.epoch_stride = stride
        self.calls_in_step = 0
        return stride % 2 == 0             # the all-gather form needs an even stride (its buffer is chosen on the host)

    def fits(self, M: int, N: int) -> bool:
        return M * ((N + 7) // 8 * 8) <= self.slot_elems and ((M + 127) // 128) * ((N + 127) // 128) <= self.max_tiles

    def _call(self, a, b, M, N, K, a_mn, b_mn, bias, out, out_dtype, mode: int = 0):
        """mode 0: all-reduce of the product; 1: reduce-scatter over rows (out has M / P rows); 2: all-gather of the
        rows of ``a`` (``a`` is this rank's M / P rows, out has M rows)."""
        from ..ops.gemm import _rowmajor

        a2, b2 = _rowmajor(a), _rowmajor(b)
        if out is None:
            out = torch.empty(M // self.P if mode == 1 else M, N, dtype=out_dtype or torch.bfloat16, device=a.device)
        self.calls_in_step += 1
        if self._step_dev is not None:
            self.ctx.epoch = self.calls_in_step
        else:
            self.epoch += 1
            self.ctx.epoch = self.epoch
        rc = _native.lib().zen_gemm_bf16_coll(_native.ptr(a2), _native.ptr(b2), _native.ptr(out), _native.ptr(bias), M, N, K,
                                              a2.stride(0), b2.stride(0), out.stride(0), int(a_mn), int(b_mn),
                                              int(out.dtype == torch.float32), 0, 0, ctypes.byref(self.ctx), mode,
                                              _native.stream_ptr())
        _native.check(rc, "zen_gemm_bf16_coll")
        return out

    def fits_rs(self, M: int, N: int) -> bool:
        rpr = M // self.P
        return (M % self.P == 0 and rpr % 128 == 0 and rpr * ((N + 7) // 8 * 8) <= self.slot_elems
                and (rpr // 128) * ((N + 127) // 128) <= self.max_tiles)

    def fits_ag(self, rows_local: int, K: int, N: int = 0) -> bool:
        """All-gather + GEMM: two ranks, whole 128-row tiles, the peer's rows fit one exchange slot; with N given also
        that the per-rank tile count fits the flag rows (the kernel takes 256-wide tiles when N allows)."""
        if not (self.P == 2 and rows_local % 128 == 0 and K % 8 == 0 and rows_local * K <= self.slot_elems):
            return False
        bn = 256 if (N >= 1024 and N % 256 == 0) else 128
        return N == 0 or (rows_local // 128) * ((N + bn - 1) // bn) <= self.max_tiles

    def gemm_rs_nt(self, a, b, bias=None, out=None):
        """reduce_scatter over rows of a[M,K] @ b[N,K]^T: this rank's M / P rows of the sum over the group (+ bias)."""
        K = a.shape[-1]
        return self._call(a, b, a.numel() // K, b.shape[0], K, False, False, bias, out, None, mode=1)

    def gemm_rs_nn(self, a, b, bias=None, out=None):
        """reduce_scatter over rows of a[M,K] @ b[K,N]."""
        K = a.shape[-1]
        return self._call(a, b, a.numel() // K, b.shape[1], K, False, True, bias, out, None, mode=1)

    def ag_gemm_nt(self, a_local, b, bias=None, out=None):
        """all_gather(a_local over rows)[M,K] @ b[N,K]^T: every rank passes its M / P rows; the kernel pushes them to the
        peer and multiplies local rows first, gathered rows as they arrive."""
        K = a_local.shape[-1]
        return self._call(a_local, b, self.P * (a_local.numel() // K), b.shape[0], K, False, False, bias, out, None, mode=2)

    def ag_gemm_nn(self, a_local, b, bias=None, out=None):
        """all_gather(a_local over rows)[M,K] @ b[K,N]."""
        K = a_local.shape[-1]
        return self._call(a_local, b, self.P * (a_local.numel() // K), b.shape[1], K, False, True, bias, out, None, mode=2)

    def gemm_ar_nt(self, a, b, bias=None, out=None):
        """all_reduce(a[M,K] @ b[N,K]^T) (+ bias, added once after the sum)."""
        K = a.shape[-1]
        return self._call(a, b, a.numel() // K, b.shape[0], K, False, False, bias, out, None)

    def gemm_ar_nn(self, a, b, bias=None, out=None):
        """all_reduce(a[M,K] @ b[K,N]) (+ bias)."""
        K = a.shape[-1]
        return self._call(a, b, a.numel() // K, b.shape[1], K, False, True, bias, out, None)

    def check(self) -> int:
        v = int(self.status.item())
        if v:
            self.status.zero_()
        return v

    def close(self):
        self.region.close()
