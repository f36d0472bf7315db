"""Tensor-parallel GEMMs with the collective fused into the kernel, against the same GEMM followed (or preceded) by
the NCCL collective, with the roofline of each: the slower of FLOPs / measured GEMM peak and bytes over NVLink / link
bandwidth.  Run under torchrun on the ranks of one TP group (2 for the all-gather mode):

    torchrun --nproc-per-node 2 bench/tp_gemm_bench.py --tokens 4096 --d 4096 --ffn 14336
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

PEAK_TFLOPS = 1377.0        # sustained bf16 matmul measured on this GPU type
LINK_GBS = 770.0            # measured peer copy, one direction


def timed(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) * 1e3            # us, max over ranks


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    from zen_repro_b200.ops import gemm as G
    from zen_repro_b200.parallel import launch_from_torch
    from zen_repro_b200.parallel.tp_fused import FusedTPWorkspace

    rank, P, dev = launch_from_torch()
    T, d, f = a.tokens, a.d, a.ffn
    ws = FusedTPWorkspace(None, T, max(d, f // P, 4096), wait_ms=2000.0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    def report(name, M, N, K, link_bytes, fused_us, split_us):
        flop_us = 2.0 * M * N * K / (PEAK_TFLOPS * 1e12) * 1e6
        link_us = link_bytes / (LINK_GBS * 1e9) * 1e6
        bound = max(flop_us, link_us)
        r = dict(op=name, M=M, N=N, K=K, ranks=P, fused_us=round(fused_us, 1), gemm_then_nccl_us=round(split_us, 1),
                 flop_bound_us=round(flop_us, 1), nvlink_bound_us=round(link_us, 1), roofline_frac=round(bound / fused_us, 3),
                 status=ws.check(), gemm_error=G.gemm_error())
        rows.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)

    # row-parallel linears (attention output, MLP down): K is sharded, the output is summed over the group
    for name, K_full in (("o_proj", d), ("mlp_down", f)):
        K = K_full // P
        x = torch.randn(T, K, device=dev).bfloat16()
        w = torch.randn(d, K, device=dev).bfloat16()
        out = torch.empty(T, d, device=dev, dtype=torch.bfloat16)

        def split_ar():
            y = G.gemm_nt(x, w, out=out)
            dist.all_reduce(y)
        report(name + " gemm+all_reduce", T, d, K, (P - 1) / P * 2 * T * d * 2, timed(lambda: ws.gemm_ar_nt(x, w), a.iters, a.warmup, flush),
               timed(split_ar, a.iters, a.warmup, flush))
        if ws.fits_rs(T, d):
            rs_out = torch.empty(T // P, d, device=dev, dtype=torch.bfloat16)

            def split_rs():
                y = G.gemm_nt(x, w, out=out)
                dist.reduce_scatter_tensor(rs_out, y)
            report(name + " gemm+reduce_scatter", T, d, K, (P - 1) / P * T * d * 2, timed(lambda: ws.gemm_rs_nt(x, w), a.iters, a.warmup, flush),
                   timed(split_rs, a.iters, a.warmup, flush))
    # column-parallel linears (qkv, gate+up) with sequence-sharded input: rows gathered, N sharded
    if P == 2:
        for name, N_full in (("qkv", d + 2 * (d // 4)), ("mlp_gate_up", 2 * f)):
            N = N_full // P
            xs = torch.randn(T // P, d, device=dev).bfloat16()
            w = torch.randn(N, d, device=dev).bfloat16()
            full = torch.empty(T, d, device=dev, dtype=torch.bfloat16)
            if not ws.fits_ag(T // P, d):
                continue

            def split_ag():
                dist.all_gather_into_tensor(full, xs)
                return G.gemm_nt(full, w)
            report(name + " all_gather+gemm", T, N, d, (P - 1) / P * T * d * 2, timed(lambda: ws.ag_gemm_nt(xs, w), a.iters, a.warmup, flush),
                   timed(split_ag, a.iters, a.warmup, flush))
    dist.barrier()
    torch.cuda.synchronize()
    ws.close()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
