"""One tcgen05 GEMM shape, a few launches: the small case for profiler captures.

    python bench/gemm_one.py --m 8192 --n 2304 --k 768 --mode nt --iters 3
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from zen_repro_b200.ops import gemm as G  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--m", type=int, default=8192)
ap.add_argument("--n", type=int, default=2304)
ap.add_argument("--k", type=int, default=768)
ap.add_argument("--mode", default="nt")
ap.add_argument("--iters", type=int, default=3)
ap.add_argument("--bn", type=int, default=0)
a = ap.parse_args()
torch.manual_seed(0)
if a.mode == "nt":
    x, w = torch.randn(a.m, a.k, device="cuda").bfloat16(), torch.randn(a.n, a.k, device="cuda").bfloat16()
    f = lambda: G.gemm_nt(x, w, bn=a.bn)
elif a.mode == "nn":
    x, w = torch.randn(a.m, a.k, device="cuda").bfloat16(), torch.randn(a.k, a.n, device="cuda").bfloat16()
    f = lambda: G.gemm_nn(x, w, bn=a.bn)
else:
    x, w = torch.randn(a.k, a.m, device="cuda").bfloat16(), torch.randn(a.k, a.n, device="cuda").bfloat16()
    f = lambda: G.gemm_tn(x, w, bn=a.bn)
for _ in range(a.iters):
    out = f()
torch.cuda.synchronize()
print("ok", float(out.float().abs().mean()), G.gemm_error())
