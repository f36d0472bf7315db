"""GEMM microbenchmark: tcgen05 kernel vs torch.matmul (cuBLAS) on the shapes of the benchmark models.

    python bench/gemm_bench.py [--shapes gpt2|llama|square] [--iters 20]
    python bench/gemm_bench.py --one 8192 2304 768 --modes nt --iters 3      # one shape, own kernel only, a few launches
                                                                             # (the small case for a profiler capture)
    python bench/gemm_bench.py --shapes gpt2 --group                         # a layer's weight gradients: 4 launches vs 1
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from zen_repro_b200.ops import gemm as G  # noqa: E402

SHAPES = {
    "gpt2": [(8192, 2304, 768), (8192, 768, 768), (8192, 3072, 768), (8192, 768, 3072), (8192, 50304, 768)],
    "gemma": [(8192, 2560, 2048), (8192, 2048, 2048), (8192, 32768, 2048), (8192, 2048, 16384)],
    "llama": [(4096, 3072, 4096), (4096, 4096, 2048), (4096, 14336, 4096), (4096, 4096, 7168)],
    "square": [(4096, 4096, 4096), (8192, 8192, 8192)],
}


# weight gradients (M = inputs, N = outputs, K = tokens) of one layer
GROUPS = {
    "gpt2": [(3072, 768, 8192), (768, 3072, 8192), (768, 768, 8192), (768, 2304, 8192)],
    "llama": [(7168, 4096, 4096), (4096, 14336, 4096), (2048, 4096, 4096), (4096, 3072, 4096)],
}


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
    ap.add_argument("--shapes", default="gpt2")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--modes", nargs="+", default=["nt", "nn", "tn"])
    ap.add_argument("--one", type=int, nargs=3, metavar=("M", "N", "K"), default=None)
    ap.add_argument("--bn", type=int, default=0, help="with --one: force the N tile (0 = chosen per call)")
    ap.add_argument("--group", action="store_true",
                    help="the weight gradients of one layer of --shapes: separate launches against one grouped launch")
    ap.add_argument("--tail_min_kb", type=int, default=-1,
                    help="fewest 64-wide K blocks from which the tiles of a partly filled last wave are cut in two "
                         "(0 = never, -1 = the library's default)")
    args = ap.parse_args()
    if args.tail_min_kb >= 0:
        from zen_repro_b200 import _native
        _native.lib().zen_gemm2_tail_split(args.tail_min_kb)
    if args.one:
        M, N, K = args.one
        torch.manual_seed(0)
        mode = args.modes[0]
        if mode == "nt":
            x, w = torch.randn(M, K, device="cuda").bfloat16(), torch.randn(N, K, device="cuda").bfloat16()
            f = lambda: G.gemm_nt(x, w, bn=args.bn)
        elif mode == "nn":
            x, w = torch.randn(M, K, device="cuda").bfloat16(), torch.randn(K, N, device="cuda").bfloat16()
            f = lambda: G.gemm_nn(x, w, bn=args.bn)
        else:
            x, w = torch.randn(K, M, device="cuda").bfloat16(), torch.randn(K, N, device="cuda").bfloat16()
            f = lambda: G.gemm_tn(x, w, bn=args.bn)
        for _ in range(args.iters):
            out = f()
        torch.cuda.synchronize()
        print("ok", float(out.float().abs().mean()), G.gemm_error())
        return
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    if args.group:
        # the weight gradients of one layer (a[K, M]^T @ b[K, N], K = tokens): one launch each, against one grouped launch
        shapes = GROUPS[args.shapes]
        ops = [(torch.randn(K, M, device="cuda").bfloat16(), torch.randn(K, N, device="cuda").bfloat16(),
                torch.empty(M, N, device="cuda", dtype=torch.bfloat16)) for (M, N, K) in shapes]

        def separate():
            for a, b, o in ops:
                G.gemm_tn(a, b, out=o)

        def grouped():
            for a, b, o in ops:
                G.defer_tn(a, b, o, False)
            G.flush_deferred()

        def library():
            for a, b, o in ops:
                torch.matmul(a.t(), b, out=o)

        old = G.GROUP_SIZE
        G.GROUP_SIZE = max(len(ops), 2)
        ts, tg, tl = bench(separate, args.iters, flush), bench(grouped, args.iters, flush), bench(library, args.iters, flush)
        G.GROUP_SIZE = old
        fl = sum(2.0 * M * N * K for (M, N, K) in shapes)
        print(json.dumps(dict(group=args.shapes, shapes=shapes, separate_ms=round(ts, 4), grouped_ms=round(tg, 4),
                              cublas_ms=round(tl, 4), separate_tflops=round(fl / ts / 1e9, 1),
                              grouped_tflops=round(fl / tg / 1e9, 1), cublas_tflops=round(fl / tl / 1e9, 1),
                              err=G.gemm_error())), flush=True)
        return
    for (M, N, K) in SHAPES[args.shapes]:
        for mode in args.modes:
            if mode == "nt":
                a = torch.randn(M, K, device="cuda").bfloat16(); b = torch.randn(N, K, device="cuda").bfloat16()
                mine, ref = (lambda: G.gemm_nt(a, b)), (lambda: a @ b.t())
            elif mode == "nn":
                a = torch.randn(M, K, device="cuda").bfloat16(); b = torch.randn(K, N, device="cuda").bfloat16()
                mine, ref = (lambda: G.gemm_nn(a, b)), (lambda: a @ b)
            else:
                a = torch.randn(K, M, device="cuda").bfloat16(); b = torch.randn(K, N, device="cuda").bfloat16()
                mine, ref = (lambda: G.gemm_tn(a, b)), (lambda: a.t() @ b)
            tm, tr = bench(mine, args.iters, flush), bench(ref, args.iters, flush)
            pair = {"nt": lambda: G.gemm_nt(a, b, bn=512), "nn": lambda: G.gemm_nn(a, b, bn=512), "tn": lambda: G.gemm_tn(a, b, bn=512)}[mode]
            one = {"nt": lambda: G.gemm_nt(a, b, bn=256), "nn": lambda: G.gemm_nn(a, b, bn=256), "tn": lambda: G.gemm_tn(a, b, bn=256)}[mode]
            tp, t1 = bench(pair, args.iters, flush), bench(one, args.iters, flush)
            fl = 2.0 * M * N * K
            print(json.dumps(dict(mode=mode, M=M, N=N, K=K, zen_ms=round(tm, 4), cublas_ms=round(tr, 4),
                                  zen_tflops=round(fl / tm / 1e9, 1), cublas_tflops=round(fl / tr / 1e9, 1),
                                  pair_tflops=round(fl / tp / 1e9, 1), one256_tflops=round(fl / t1 / 1e9, 1),
                                  err=G.gemm_error())), flush=True)


if __name__ == "__main__":
    main()
