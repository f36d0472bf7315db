"""The allocation-free column sum, called through its exported C symbol.

Some callers of this library may not allocate device memory at the call site: a host that has given all
device memory to its own pool, a callback in which the allocator must not be re-entered, a plain C
program without torch's allocator.  ``zen_colsum_noalloc`` serves them with scratch that lives inside the
library.  This test checks it against the regular entry point (``zen_colsum``, caller-provided scratch) on
two calls in a row, which also shows that the shared scratch needs no clearing between calls, and checks
that an oversized request is refused before anything is launched.  It is collected last on purpose: a run
that stops at the first failure has then already covered every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from zen_repro_b200 import build

    path = build.lib_path()
    if not path.exists():
        path = build.build()
    lib = ctypes.CDLL(str(path))
    lib.zen_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _reference(lib, a, accumulate_into=None):
    rows, cols = a.shape
    parts = lib.zen_colsum_parts(rows)
    scratch = torch.empty(parts * cols, dtype=torch.float32, device=a.device)
    out = accumulate_into.clone() if accumulate_into is not None else torch.empty(cols, dtype=a.dtype, device=a.device)
    code = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[a.dtype]
    rc = lib.zen_colsum(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(scratch.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                        rows, cols, int(accumulate_into is not None), code,
                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_matches_regular_entry_point_twice(dtype):
    lib = _lib()
    dev = torch.device("cuda")
    code = {torch.float32: 0, torch.bfloat16: 1}[dtype]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.manual_seed(0)
    # two different shapes back to back: the second call sees the first call's leftovers in the scratch
    for rows, cols in [(4096, 768), (1000, 3072)]:
        a = torch.randn(rows, cols, device=dev).to(dtype)
        out = torch.empty(cols, dtype=dtype, device=dev)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = lib.zen_colsum_noalloc(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(out.data_ptr()), rows, cols, 0, code, stream)
        assert rc == 0, lib.zen_noalloc_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        want = _reference(lib, a)
        tol = dict(atol=1e-4, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.3, rtol=2e-2)
        torch.testing.assert_close(out.float(), want.float(), **tol)
        torch.testing.assert_close(out.float(), a.float().sum(0), **tol)
        # accumulate form
        base = torch.randn(cols, device=dev).to(dtype)
        acc = base.clone()
        rc = lib.zen_colsum_noalloc(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(acc.data_ptr()), rows, cols, 1, code, stream)
        assert rc == 0, lib.zen_noalloc_last_error()
        torch.testing.assert_close(acc.float(), _reference(lib, a, base).float(), **tol)


def test_noalloc_refuses_oversized_and_bad_arguments():
    lib = _lib()
    dev = torch.device("cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    a = torch.zeros(8, 8, device=dev)
    out = torch.full((8,), 7.0, device=dev)
    # 65536 rows x 4096 cols would need 2048 * 4096 floats of scratch: more than the built-in 2**20
    rc = lib.zen_colsum_noalloc(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(out.data_ptr()), 65536, 4096, 0, 0, stream)
    assert rc == -20 and b"scratch" in lib.zen_noalloc_last_error()
    rc = lib.zen_colsum_noalloc(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(out.data_ptr()), 8, 12, 0, 0, stream)
    assert rc == -21
    torch.cuda.synchronize()
    assert float(out.sum()) == 56.0          # nothing was launched
