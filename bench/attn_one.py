"""One attention shape, forward and backward once or a few times: the small case for profiler captures.

    python bench/attn_one.py --b 8 --s 1024 --hq 12 --hkv 12 --hd 64 --iters 2
"""
import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from zen_repro_b200.ops import attention as A  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--b", type=int, default=8)
ap.add_argument("--s", type=int, default=1024)
ap.add_argument("--hq", type=int, default=12)
ap.add_argument("--hkv", type=int, default=12)
ap.add_argument("--hd", type=int, default=64)
ap.add_argument("--iters", type=int, default=2)
a = ap.parse_args()
torch.manual_seed(0)
qkv = (torch.randn(a.b * a.s, (a.hq + 2 * a.hkv) * a.hd, device="cuda") * 0.5).bfloat16()
do = (torch.randn(a.b * a.s, a.hq * a.hd, device="cuda") * 0.5).bfloat16()
sc = 1 / math.sqrt(a.hd)
for _ in range(a.iters):
    out, lse = A.attention_fwd_kernel(qkv, a.b, a.s, a.hq, a.hkv, a.hd, sc)
    if a.hd <= 256:
        dq = A.attention_bwd_kernel(do, qkv, out, lse, a.b, a.s, a.hq, a.hkv, a.hd, sc)
torch.cuda.synchronize()
print("ok", float(out.float().abs().mean()), A.attention_error())
