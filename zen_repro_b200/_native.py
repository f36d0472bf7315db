"""ctypes access to the in-tree native library (``_lib/libzen_b200.so``).

The library is plain CUDA with a C ABI: every entry point takes raw device
pointers, sizes and a ``cudaStream_t``.  ``lib()`` loads it once; on a machine
with a GPU a missing library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

import torch

from . import build as _build

_LOCK = threading.Lock()
_LIB: ctypes.CDLL | None = None


class NativeUnavailable(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
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
            _LIB = ctypes.CDLL(str(path))
    return _LIB


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
