"""GEMM entry points.  bf16 CUDA operands run the tcgen05 kernel (csrc/gemm_tcgen05.cu); everything
else (CPU, fp32) runs ``torch.matmul`` and doubles as the oracle in tests.

Naming: ``nt`` = A[M,K] @ B[N,K]^T, ``nn`` = A[M,K] @ B[K,N], ``tn`` = A[K,M]^T @ B[K,N].  These are the
forward, input-gradient and weight-gradient products of a linear layer (in either weight layout), so
no operand is ever transposed in memory.
"""
from __future__ import annotations

import os

import torch

from .. import _native

_FORCE_TORCH = os.environ.get("ZEN_GEMM", "") == "torch"
_PAIR_MODE = os.environ.get("ZEN_GEMM_2CTA", "auto")      # auto | 0 | 1


def use_pair_kernel(M: int, N: int, K: int) -> bool:
    """CTA-pair (256 x 256 tile) kernel when the problem fills the 74 clusters reasonably well."""
    if _PAIR_MODE == "0":
        return False
    if _PAIR_MODE == "1":
        return M >= 256 and N >= 128
    if M < 512 or N < 256:
        return False
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    waves = -(-tiles // 74)
    eff = tiles / (waves * 74.0)
    pad = (N / (((N + 255) // 256) * 256.0)) * (M / (((M + 255) // 256) * 256.0))
    score = eff * pad
    return score >= 0.8 or (score >= 0.6 and K >= 1024)


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


def _launch(a, b, M, N, K, a_mn, b_mn, bias, out, accumulate, out_dtype, bn):
    a2, b2 = _rowmajor(a), _rowmajor(b)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=a.device)
        accumulate = False
    assert out.dim() == 2 and out.shape == (M, N) and out.stride(1) == 1
    assert out.dtype in (torch.bfloat16, torch.float32)
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.is_contiguous() and bias.numel() == N
    pair = (bn == 512) or (bn == 0 and use_pair_kernel(M, N, K))
    if pair:
        rc = _native.lib().zen_gemm_bf16_2cta(_native.ptr(a2), _native.ptr(b2), _native.ptr(out), _native.ptr(bias), M, N, K,
                                              a2.stride(0), b2.stride(0), out.stride(0), int(a_mn), int(b_mn),
                                              int(out.dtype == torch.float32), int(accumulate), _native.stream_ptr())
        _native.check(rc, "zen_gemm_bf16_2cta")
        return out
    rc = _native.lib().zen_gemm_bf16(_native.ptr(a2), _native.ptr(b2), _native.ptr(out), _native.ptr(bias), M, N, K,
                                     a2.stride(0), b2.stride(0), out.stride(0), int(a_mn), int(b_mn),
                                     int(out.dtype == torch.float32), int(accumulate), bn, _native.stream_ptr())
    _native.check(rc, "zen_gemm_bf16")
    return out


def gemm_nt(a, b, bias=None, out=None, accumulate=False, out_dtype=None, bn=0):
    """a[M,K] @ b[N,K]^T (+ bias[N])."""
    M, K = a.shape[-2] if a.dim() == 2 else a.numel() // a.shape[-1], a.shape[-1]
    N = b.shape[0]
    if not _use_kernel(a, b):
        r = a.reshape(-1, K).float() @ b.float().t()
        return _finish(r, bias, out, accumulate, out_dtype or a.dtype)
    return _launch(a, b, M, N, K, False, False, bias, out, accumulate, out_dtype, bn)


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
