"""GEMM entry points.  bf16 CUDA operands run the tcgen05 kernel (csrc/gemm_tcgen05.cu); everything
else (CPU, fp32) runs ``torch.matmul`` and doubles as the oracle in tests.

Naming: ``nt`` = A[M,K] @ B[N,K]^T, ``nn`` = A[M,K] @ B[K,N], ``tn`` = A[K,M]^T @ B[K,N].  These are the
forward, input-gradient and weight-gradient products of a linear layer (in either weight layout), so
no operand is ever transposed in memory.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _native

_FORCE_TORCH = os.environ.get("ZEN_GEMM", "") == "torch"
_PAIR_MODE = os.environ.get("ZEN_GEMM_2CTA", "auto")      # auto | 0 | 1


_clusters_cached = [0]


def _clusters() -> int:
    """CTA pairs the device runs at once (one per two SMs; 74 on a B200)."""
    if not _clusters_cached[0]:
        n = 148
        if torch.cuda.is_available():
            n = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        _clusters_cached[0] = max(1, n // 2)
    return _clusters_cached[0]


def use_pair_kernel(M: int, N: int, K: int) -> bool:
    """CTA-pair (256 x 256 tile) kernel when the problem fills the 74 clusters reasonably well."""
    if _PAIR_MODE == "0":
        return False
    if _PAIR_MODE == "1":
        return M >= 256 and N >= 128
    if M < 512 or N < 256:
        return False
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    waves = -(-tiles // _clusters())
    eff = tiles / float(waves * _clusters())
    pad = (N / (((N + 255) // 256) * 256.0)) * (M / (((M + 255) // 256) * 256.0))
    score = eff * pad
    return score >= 0.6


_SPLITK = os.environ.get("ZEN_GEMM_SPLITK", "auto")       # auto | 0
_TAIL_SPLIT = os.environ.get("ZEN_GEMM_TAILSPLIT", "1") != "0"
_WS_FLOATS = 74 * 2 * 128 * 256                            # one fp32 partial tile per CTA of one full wave
_N_COUNTERS = 4096
_ws_cache: dict = {}
# below this K the extra pass over the partial tiles costs more than the idle clusters
_SPLITK_MIN_K = int(os.environ.get("ZEN_GEMM_SPLITK_MIN_K", "4096"))


def split_k_choice(M: int, N: int, K: int) -> int:
    """Number of K slices for the CTA-pair kernel, or 1.  Splitting pays when the output has far fewer 256 x 256
    tiles than the 74 clusters and K is long: the weight-gradient products of a transformer layer."""
    if _SPLITK == "0" or _PAIR_MODE == "0" or M < 256 or N < 256 or K < _SPLITK_MIN_K:
        return 1
    tm, tn = (M + 255) // 256, (N + 255) // 256
    tiles = tm * tn
    # both slices of every tile must be resident in the launch's single wave of clusters (they wait for each other)
    if (M * N) / (tiles * 65536.0) < 0.75 or tiles * 2 > _clusters():
        return 1
    splits = min(_clusters() // tiles, (K // 64) // 8, 2)  # two slices: the fast store path of the kernel
    return splits if splits >= 2 and tiles * splits * 2 * 128 * 256 <= _WS_FLOATS and tiles * 16 <= _N_COUNTERS else 1


def _splitk_workspace(device):
    """fp32 partial tiles and arrival counters for the split-K kernel, one pair per device and stream: the
    kernel's slices meet through them, so two launches may share them only in stream order."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    w = _ws_cache.get(key)
    if w is None:
        w = (torch.empty(_WS_FLOATS, dtype=torch.float32, device=device),
             torch.zeros(_N_COUNTERS, dtype=torch.int32, device=device))
        _ws_cache[key] = w
    return w


def _use_kernel(a: torch.Tensor, b: torch.Tensor) -> bool:
    return (a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and not _FORCE_TORCH)


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
    """2-D view with unit inner stride, 16-byte aligned base and row stride a multiple of 8."""
    if t.dim() != 2:
        t = t.reshape(-1, t.shape[-1])
    if t.stride(1) != 1 or t.stride(0) % 8 or t.data_ptr() % 16 or (t.shape[0] > 1 and t.stride(0) < t.shape[1]):
        cols = t.shape[1]
        pad = (-cols) % 8
        t = torch.nn.functional.pad(t, (0, pad))[:, :cols] if pad else t.contiguous()
    return t


def _launch(a, b, M, N, K, a_mn, b_mn, bias, out, accumulate, out_dtype, bn, pad_ok=False):
    a2, b2 = _rowmajor(a), _rowmajor(b)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=a.device)
        accumulate = False
    assert out.dim() == 2 and out.shape == (M, N) and out.stride(1) == 1
    assert out.dtype in (torch.bfloat16, torch.float32)
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.is_contiguous() and bias.numel() == N
    splits = split_k_choice(M, N, K) if bn == 0 else 1
    if splits > 1:
        ws, cnt = _splitk_workspace(a.device)
        rc = _native.lib().zen_gemm_bf16_2cta_splitk(
            _native.ptr(a2), _native.ptr(b2), _native.ptr(out), _native.ptr(bias), M, N, K, a2.stride(0), b2.stride(0),
            out.stride(0), int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate), splits,
            _native.ptr(ws), ctypes.c_uint64(ws.numel()), _native.ptr(cnt), cnt.numel(), 0, _native.stream_ptr())
        _native.check(rc, "zen_gemm_bf16_2cta_splitk")
        return out
    pair = (bn == 512) or (bn == 0 and use_pair_kernel(M, N, K))
    if pair:
        n_store = min((N + 7) // 8 * 8, out.stride(0)) if pad_ok else 0
        # the workspace lets the launcher cut the tiles of a partly filled last wave of clusters into two K slices
        ws, cnt = _splitk_workspace(a.device) if _TAIL_SPLIT else (None, None)
        rc = _native.lib().zen_gemm_bf16_2cta_splitk(
            _native.ptr(a2), _native.ptr(b2), _native.ptr(out), _native.ptr(bias), M, N, K, a2.stride(0), b2.stride(0),
            out.stride(0), int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate), 1,
            _native.ptr(ws), ctypes.c_uint64(ws.numel() if ws is not None else 0), _native.ptr(cnt),
            cnt.numel() if cnt is not None else 0, n_store, _native.stream_ptr())
        _native.check(rc, "zen_gemm_bf16_2cta")
        return out
    rc = _native.lib().zen_gemm_bf16(_native.ptr(a2), _native.ptr(b2), _native.ptr(out), _native.ptr(bias), M, N, K,
                                     a2.stride(0), b2.stride(0), out.stride(0), int(a_mn), int(b_mn),
                                     int(out.dtype == torch.float32), int(accumulate), bn, _native.stream_ptr())
    _native.check(rc, "zen_gemm_bf16")
    return out


def gemm_nt(a, b, bias=None, out=None, accumulate=False, out_dtype=None, bn=0, pad_ok=False):
    """a[M,K] @ b[N,K]^T (+ bias[N]).  ``pad_ok``: ``out`` is the first N columns of a wider buffer whose columns up to
    the next multiple of 8 may be overwritten (with zeros); lets an odd N use the full-line store path."""
    M, K = a.shape[-2] if a.dim() == 2 else a.numel() // a.shape[-1], a.shape[-1]
    N = b.shape[0]
    if not _use_kernel(a, b):
        r = a.reshape(-1, K).float() @ b.float().t()
        return _finish(r, bias, out, accumulate, out_dtype or a.dtype)
    return _launch(a, b, M, N, K, False, False, bias, out, accumulate, out_dtype, bn, pad_ok)


def gemm_nn(a, b, bias=None, out=None, accumulate=False, out_dtype=None, bn=0):
    """a[M,K] @ b[K,N] (+ bias[N])."""
    K = a.shape[-1]
    M = a.numel() // K
    N = b.shape[1]
    if not _use_kernel(a, b):
        r = a.reshape(-1, K).float() @ b.float()
        return _finish(r, bias, out, accumulate, out_dtype or a.dtype)
    return _launch(a, b, M, N, K, False, True, bias, out, accumulate, out_dtype, bn)


def gemm_tn(a, b, out=None, accumulate=False, out_dtype=None, bn=0):
    """a[K,M]^T @ b[K,N]: the weight-gradient product (sum over tokens)."""
    M, N = a.shape[-1], b.shape[-1]
    K = a.numel() // M
    if not _use_kernel(a, b):
        r = a.reshape(-1, M).float().t() @ b.reshape(-1, N).float()
        return _finish(r, None, out, accumulate, out_dtype or a.dtype)
    return _launch(a, b, M, N, K, True, True, None, out, accumulate, out_dtype, bn)


# ---------------------------------------------------------------------------------------------------------------
# Deferred weight gradients.  The weight-gradient products of a transformer layer are small (27 / 9 / 36 / 36 output
# tiles for GPT-2 small against 74 CTA pairs) and nothing downstream in backward waits for them, so a linear layer's
# backward may queue its product here instead of launching it; GROUP_SIZE queued products (or the end of the backward
# pass, or an explicit flush) go out as ONE launch whose clusters walk the tiles of all of them.
class _GemmDesc(ctypes.Structure):
    _fields_ = [("A", ctypes.c_void_p), ("B", ctypes.c_void_p), ("C", ctypes.c_void_p),
                ("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32),
                ("lda", ctypes.c_int32), ("ldb", ctypes.c_int32), ("ldc", ctypes.c_int32),
                ("out_fp32", ctypes.c_int32), ("accumulate", ctypes.c_int32)]


GROUP_SIZE = int(os.environ.get("ZEN_GEMM_GROUP", "4"))      # 0 / 1 = launch every weight gradient by itself
_pending: list = []
_callback_armed = [False]


def defer_tn(a, b, out, accumulate: bool, done=None) -> None:
    """Queue ``out (+)= a[K,M]^T @ b[K,N]`` (bf16 CUDA operands, ``out`` a 2-D bf16 / fp32 tensor with unit inner stride);
    ``done()`` runs right after the launch that contains it has been enqueued.  Falls back to an immediate
    :func:`gemm_tn` when grouping is off or the operands do not qualify."""
    M, N = a.shape[-1], b.shape[-1]
    K = a.numel() // M
    # products with many tiles fill the clusters by themselves; grouping them only delays their gradient
    small = ((M + 255) // 256) * ((N + 255) // 256) <= 2 * _clusters()
    ok = (GROUP_SIZE > 1 and small and _use_kernel(a, b) and _PAIR_MODE != "0" and M >= 256 and N >= 256 and out.is_cuda
          and out.dim() == 2 and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32))
    if not ok:
        gemm_tn(a, b, out=out, accumulate=accumulate)
        if done is not None:
            done()
        return
    if any(item[2].data_ptr() == out.data_ptr() for item in _pending):
        flush_deferred()                           # two products into one output never share a launch
    a2, b2 = _rowmajor(a), _rowmajor(b)
    _pending.append((a2, b2, out, M, N, K, bool(accumulate), done))
    arm_flush_at_end_of_backward()
    if len(_pending) >= GROUP_SIZE:
        flush_deferred()


def arm_flush_at_end_of_backward() -> bool:
    """Ask the autograd engine to call :func:`flush_deferred` when the running backward pass ends.  False when no
    backward pass is running (the caller then flushes, or does not defer)."""
    if not _callback_armed[0]:
        try:
            torch.autograd.Variable._execution_engine.queue_callback(flush_deferred)
            _callback_armed[0] = True
        except RuntimeError:
            return False
    return True


def flush_deferred() -> None:
    """Launch whatever :func:`defer_tn` has queued (one launch per GROUP_SIZE products) and run the callbacks."""
    _callback_armed[0] = False
    while _pending:
        batch = _pending[:min(max(GROUP_SIZE, 1), _native.lib().zen_gemm_group_max())]
        del _pending[:len(batch)]
        lib = _native.lib()
        n = len(batch)
        descs = (_GemmDesc * n)()
        for i, (a2, b2, out, M, N, K, acc, _done) in enumerate(batch):
            descs[i] = _GemmDesc(a2.data_ptr(), b2.data_ptr(), out.data_ptr(), M, N, K, a2.stride(0), b2.stride(0),
                                 out.stride(0), int(out.dtype == torch.float32), int(acc))
        dev = batch[0][0].device
        ws, cnt = _splitk_workspace(dev) if _TAIL_SPLIT else (None, None)
        rc = lib.zen_gemm_bf16_2cta_group(descs, n, 1, 1, _native.ptr(ws), ctypes.c_uint64(ws.numel() if ws is not None else 0),
                                          _native.ptr(cnt), cnt.numel() if cnt is not None else 0, _native.stream_ptr())
        _native.check(rc, "zen_gemm_bf16_2cta_group")
        for item in batch:
            if item[7] is not None:
                item[7]()
    from . import elementwise as _E

    _E.flush_colreduce()                           # the bias / norm-parameter reductions queued beside them


def _finish(r, bias, out, accumulate, dtype):
    if bias is not None:
        r = r + bias.float()
    if out is not None:
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r.to(out.dtype))
        return out
    return r.to(dtype)


def gemm_error() -> int:
    """Error code of the last tcgen05 kernel that gave up a bounded wait (0 = none)."""
    lib = _native.lib()
    return int(lib.zen_gemm_error()) or int(lib.zen_gemm2_error())
