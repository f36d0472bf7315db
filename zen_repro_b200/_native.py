"""ctypes access to the in-tree native library (``_lib/libzen_b200.so``).

The library is plain CUDA with a C ABI: every entry point takes raw device
pointers, sizes and a ``cudaStream_t``.  ``lib()`` loads it once; on a machine
with a GPU a missing library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import threading

import torch

from . import build as _build

_LOCK = threading.Lock()
_LIB = None


class NativeUnavailable(RuntimeError):
    pass


# kernels launched by one call of each entry point (entries not listed launch one, helpers launch none)
KERNELS_PER_CALL = {
    "zen_gather_push": 1, "zen_densify": 2, "zen_sparse_allreduce": 5, "zen_sample_exchange": 2, "zen_sample_xchg_size": 0, "zen_mc_ar_ctx_size": 0, "zen_norm_bwd": 2, "zen_colsum": 2, "zen_embedding_bwd_rows": 5,
    "zen_row_gather_push": 2, "zen_attn_bwd": 3, "zen_attn_error": 0, "zen_attn_bwd64_variant": 0, "zen_gemm2_force_bn": 0, "zen_gemm2_tail_split": 0, "zen_gemm_desc_size": 0, "zen_gemm_group_max": 0, "zen_act_bwd_colsum": 1, "zen_act_colsum_parts": 0, "zen_colsum_reduce": 1, "zen_colsum_partial": 1, "zen_colreduce_multi": 1, "zen_colreduce_job_size": 0, "zen_colreduce_max_jobs": 0, "zen_norm_bwd_parts_used": 0, "zen_norm_bwd_ex": 2, "zen_select_kth": 7, "zen_gemm2_error": 0, "zen_gemm_ar_ctx_size": 0, "zen_sparse_ctx_size": 0, "zen_row_ctx_size": 0, "zen_adam_tensor_size": 0,
    "zen_norm_bwd_parts": 0, "zen_colsum_parts": 0, "zen_gemm_error": 0, "zen_sym_alloc": 0, "zen_sym_free": 0,
    "zen_ipc_get_handle": 0, "zen_ipc_open": 0, "zen_ipc_close": 0, "zen_enable_peer": 0, "zen_ipc_handle_size": 0,
}


class _CountingLib:
    """Proxy over the CDLL that counts kernel launches issued through it (read by the benchmark)."""

    def __init__(self, cdll: ctypes.CDLL):
        self._cdll = cdll
        self.launches = 0
        self._cache: dict = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._cdll, name)
            n = KERNELS_PER_CALL.get(name, 1)
            if n == 0:
                fn = raw
            else:
                def fn(*a, _raw=raw, _n=n, _self=self):
                    _self.launches += _n
                    return _raw(*a)
            self._cache[name] = fn
        return fn


def lib() -> "_CountingLib":
    """The loaded native library; builds it first if the ``.so`` is missing and nvcc exists."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is None:
            path = _build.lib_path()
            if not path.exists():
                try:
                    path = _build.build()
                except Exception as e:  # pragma: no cover - depends on toolchain
                    raise NativeUnavailable(f"native library missing and build failed: {e}") from e
            _LIB = _CountingLib(ctypes.CDLL(str(path)))
    return _LIB


def launch_count() -> int:
    """Kernels of this library launched so far in this process."""
    return _LIB.launches if _LIB is not None else 0


def available() -> bool:
    """True when CUDA kernels can run here (a GPU is present and the library loads)."""
    if not torch.cuda.is_available():
        return False
    lib()
    return True


def stream_ptr(stream: torch.cuda.Stream | None = None) -> ctypes.c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with CUDA/launcher code {rc}")
