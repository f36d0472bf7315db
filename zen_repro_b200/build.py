"""In-tree build of the native library: plain ``nvcc`` for sm_100a, no torch headers.

Every ``.cu`` under ``csrc/`` is compiled to an object (in parallel, cached by
source hash) and linked into ``zen_repro_b200/_lib/libzen_b200.so``, which the
Python side opens with ``ctypes``.  The kernels take raw device pointers and a
stream, so the library has no dependency on libtorch and builds in seconds.

    python -m zen_repro_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "_lib"
LIBNAME = "libzen_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _compile_one(src: Path, verbose: bool) -> tuple[Path, str]:
    obj = LIBDIR / f"{src.stem}.{_digest(src)}.o"
    log = ""
    if not obj.exists():
        for old in LIBDIR.glob(f"{src.stem}.*.o"):
            old.unlink()
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = r.stdout + r.stderr
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{log}")
        (LIBDIR / f"{src.stem}.ptxas.log").write_text(log)
    return obj, log


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile and link the native library; returns the path of the ``.so``."""
    LIBDIR.mkdir(exist_ok=True)
    if force:
        for f in LIBDIR.glob("*.o"):
            f.unlink()
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as ex:
        results = list(ex.map(lambda s: _compile_one(s, verbose), srcs))
    objs = [o for o, _ in results]
    out = LIBDIR / LIBNAME
    stamp = LIBDIR / "link.stamp"
    want = " ".join(o.name for o in objs)
    if force or not out.exists() or not stamp.exists() or stamp.read_text() != want:
        cmd = [_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
        stamp.write_text(want)
    if verbose:
        for _, log in results:
            if log:
                print(log)
    return out


def lib_path() -> Path:
    return LIBDIR / LIBNAME


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(p)
