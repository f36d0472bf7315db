"""Multi-GPU checks (one process per GPU over NVLink peer memory).  Skipped with fewer than two GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(names, nproc, timeout=600):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", "29617", os.path.join(HERE, "multigpu_worker.py"), *names]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


@pytest.mark.parametrize("name", ["sparse", "b2b", "samples", "nvls", "nvls_dense", "verify", "rows", "trainer", "hook", "departed", "gemm_ar", "gemm_rs_ag",
                                  "tp_trainer", "sp_trainer", "tp2dp2"])
def test_multigpu(name):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    if name == "tp2dp2" and n < 4:
        pytest.skip("needs four GPUs")
    nproc = 2 if name in ("departed", "verify", "samples", "gemm_ar", "gemm_rs_ag", "tp_trainer", "sp_trainer") else min(n, 4)
    out = _run([name], nproc)
    assert out.count("OK ") >= nproc, out
