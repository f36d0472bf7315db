"""Attention microbenchmark: the tcgen05 flash kernels (forward, backward) against the library flash attention
(``torch.nn.functional.scaled_dot_product_attention``) on the shapes of the benchmark models.

    python bench/attention_bench.py [--shapes gpt2 llama gemma opt] [--iters 20]
    python bench/attention_bench.py --one 8 1024 12 12 64 --iters 2     # B S Hq Hkv hd: own kernels only, a few launches
                                                                        # (the small case for a profiler capture)
"""
import argparse
import json
import math
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from zen_repro_b200.ops import attention as A  # noqa: E402

SHAPES = {"gpt2": (8, 1024, 12, 12, 64), "llama": (1, 4096, 32, 8, 128), "gemma": (4, 2048, 8, 1, 256), "opt": (4, 1024, 32, 32, 80)}


def bench(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record(); torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", nargs="+", default=["gpt2", "llama", "gemma"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--one", type=int, nargs=5, metavar=("B", "S", "HQ", "HKV", "HD"), default=None)
    args = ap.parse_args()
    torch.manual_seed(0)
    if args.one:
        b, s, hq, hkv, hd = args.one
        qkv = (torch.randn(b * s, (hq + 2 * hkv) * hd, device="cuda") * 0.5).bfloat16()
        do = (torch.randn(b * s, hq * hd, device="cuda") * 0.5).bfloat16()
        for _ in range(args.iters):
            out, lse = A.attention_fwd_kernel(qkv, b, s, hq, hkv, hd, 1 / math.sqrt(hd))
            A.attention_bwd_kernel(do, qkv, out, lse, b, s, hq, hkv, hd, 1 / math.sqrt(hd))
        torch.cuda.synchronize()
        print("ok", float(out.float().abs().mean()), A.attention_error())
        return
    from zen_repro_b200.ops import autograd as O

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name in args.shapes:
        b, s, hq, hkv, hd = SHAPES[name]
        sc = 1 / math.sqrt(hd)
        qkv = (torch.randn(b * s, (hq + 2 * hkv) * hd, device="cuda") * 0.5).bfloat16().requires_grad_(True)
        do = (torch.randn(b * s, hq * hd, device="cuda") * 0.5).bfloat16()
        if A.have_kernel(s, hq, hkv, hd, qkv.dtype):                # the kernels themselves, as the training step calls them
            qd = qkv.detach()
            own_out, lse = A.attention_fwd_kernel(qd, b, s, hq, hkv, hd, sc)
            t_fwd = bench(lambda: A.attention_fwd_kernel(qd, b, s, hq, hkv, hd, sc), args.iters, flush)
            t_bwd = bench(lambda: A.attention_bwd_kernel(do, qd, own_out, lse, b, s, hq, hkv, hd, sc), args.iters, flush)
        else:                                                       # padded shapes go through the autograd wrapper
            own_out = O.attention(qkv, b, s, hq, hkv, hd)
            t_fwd = bench(lambda: O.attention(qkv.detach(), b, s, hq, hkv, hd), args.iters, flush)
            t_bwd = bench(lambda: torch.autograd.grad(own_out, qkv, do, retain_graph=True), args.iters, flush)
        q, k, v = A._split(qkv, b, s, hq, hkv, hd)
        lib_out = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=sc, enable_gqa=(hq != hkv))
        dl = do.view(b, s, hq, hd).transpose(1, 2)
        l_fwd = bench(lambda: F.scaled_dot_product_attention(q.detach(), k.detach(), v.detach(), is_causal=True, scale=sc,
                                                             enable_gqa=(hq != hkv)), args.iters, flush)
        l_bwd = bench(lambda: torch.autograd.grad(lib_out, qkv, dl, retain_graph=True), args.iters, flush)
        fl = 4.0 * b * hq * s * s * hd / 2                        # causal: half of the score matrix
        print(json.dumps(dict(shape=name, B=b, S=s, hq=hq, hkv=hkv, hd=hd, fwd_us=round(t_fwd * 1e3, 1), bwd_us=round(t_bwd * 1e3, 1),
                              lib_fwd_us=round(l_fwd * 1e3, 1), lib_bwd_us=round(l_bwd * 1e3, 1),
                              fwd_tflops=round(fl / t_fwd / 1e9, 1), bwd_tflops=round(2.5 * fl / t_bwd / 1e9, 1),
                              err=A.attention_error())), flush=True)


if __name__ == "__main__":
    main()
