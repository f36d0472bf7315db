"""Sparse all-reduce microbenchmark: device time per call, effective bandwidth, stage breakdown.

Single GPU (``--virtual P``): all ranks on one device, phase by phase -- measures the kernels without
NVLink.  Multi GPU (under torchrun): one process per GPU, P2P stores over NVLink, compared with the
dense NCCL all-reduce of the same bucket.  Times are CUDA events, max over ranks.

    python bench/sparse_microbench.py --virtual 8 --log2n 24 --density 0.01
    torchrun --nproc-per-node 8 bench/sparse_microbench.py --log2n 26 28 --density 0.001 0.01 0.05 0.1
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_inputs(n, density, P, dtype, dev, dist_kind, overlap, seed=0):
    """Per-rank sparse tensors; ``overlap`` = fraction of each rank's index set drawn from a shared pool."""
    outs = []
    k = max(1, int(n * density))
    g = torch.Generator(device=dev).manual_seed(seed)
    def draw(cnt, gen):
        if dist_kind == "zipf":
            u = torch.rand(cnt, device=dev, generator=gen, dtype=torch.float64)
            # inverse-CDF of a continuous power law with exponent 1.2 truncated to [1, n]
            a = 1.2
            x = (1 - u * (1 - float(n) ** (1 - a))) ** (1 / (1 - a))
            return (x.long() - 1).clamp_(0, n - 1)
        return torch.randint(0, n, (cnt,), device=dev, generator=gen)
    shared = draw(int(k * overlap), g)
    for r in range(P):
        gr = torch.Generator(device=dev).manual_seed(seed * 1000 + r + 1)
        own = draw(k - shared.numel(), gr)
        idx = torch.cat([shared, own])
        x = torch.zeros(n, dtype=dtype, device=dev)
        x[idx] = torch.randn(idx.numel(), device=dev, generator=gr).to(dtype)
        outs.append(x)
    return outs


def time_fn(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--virtual", type=int, default=0)
    ap.add_argument("--log2n", type=int, nargs="+", default=[24])
    ap.add_argument("--density", type=float, nargs="+", default=[0.01])
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--dist", default="uniform", choices=["uniform", "zipf"])
    ap.add_argument("--overlap", type=float, default=0.0)
    ap.add_argument("--method", default="auto")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default=None)
    ap.add_argument("--plan_methods", type=int, nargs="+", default=[3],
                    help="methods the buffers are sized for (1 needs record slots for a full sparse all-gather)")
    ap.add_argument("--transport", default="p2p", choices=["p2p", "nvls"],
                    help="gather push: one store per peer, or one multimem store replicated by the NVSwitch")
    ap.add_argument("--with_reference", action="store_true",
                    help="also time the reference's own zen_sparse_comm (NCCL + its kernels, bf16 only) from baseline/_ref")
    args = ap.parse_args()
    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32}[args.dtype]
    method = int(args.method) if args.method.isdigit() else args.method
    from zen_repro_b200.sparse import engine as E

    rows = []
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.virtual or world == 1:
        P = args.virtual or 1
        dev = torch.device("cuda:0")
        torch.cuda.set_device(dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        for ln in args.log2n:
            n = 1 << ln
            for d in args.density:
                eng = E.VirtualSparseAllReduce(n, P, max_density=max(0.02, d * 1.5), methods=tuple(args.plan_methods))
                xs = make_inputs(n, d, P, dtype, dev, args.dist, args.overlap)
                ms = time_fn(lambda: eng(xs, method=method), args.iters, args.warmup, flush)
                st = eng.status()
                # stage breakdown on rank 0's kernels
                stages = {}
                r0 = eng.ranks
                def stage(name, f):
                    stages[name] = time_fn(f, 5, 1, flush)
                eng.epoch += 1; e = eng.epoch
                stage("partition_push_all", lambda: [r.partition_push(x, e) for r, x in zip(r0, xs)])
                stage("owner_reduce_all", lambda: [r.owner_reduce(e, dtype) for r in r0])
                stage("reduce_plus_gather_all", lambda: ([r.owner_reduce(e, dtype) for r in r0], [r.gather_push(e, dtype) for r in r0]))
                [r.owner_reduce(e, dtype) for r in r0]; [r.gather_push(e, dtype) for r in r0]
                out = torch.empty_like(xs[0])
                stage("densify_one", lambda: r0[0].densify(out, e))
                eng.status()
                outs = eng(xs, method=method)
                want = torch.zeros(n, dtype=torch.float32, device=dev)
                for x in xs:
                    want += x.float()
                err = max(float((o.float() - want).abs().max()) for o in outs)
                st = [a | b for a, b in zip(st, eng.status())]
                row = dict(mode="virtual", max_err=err, P=P, log2n=ln, density=d, dtype=args.dtype, dist=args.dist,
                           overlap=args.overlap, method=str(method), ms_all_ranks=ms, ms_per_rank=ms / P,
                           dense_bytes=n * xs[0].element_size(), status=st, stages_ms=stages)
                rows.append(row)
                print(json.dumps(row), flush=True)
                del eng, xs
                torch.cuda.empty_cache()
    else:
        import torch.distributed as dist

        rank = int(os.environ["RANK"]); local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dev = torch.device(f"cuda:{local}")
        dist.init_process_group("nccl", device_id=dev)
        P = world
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        ref_lba = None
        if args.with_reference and dtype == torch.bfloat16:
            root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
            sys.path.insert(0, os.path.join(root, "baseline", "shims"))
            sys.path.insert(0, os.path.join(root, "baseline", "_ref"))
            try:
                import logging

                import comm as ref_comm

                ref_lba = ref_comm.LoadBalanceAllreduce(dist.group.WORLD, list(range(world)), logging.getLogger("ref"))
            except Exception as ex:  # reference not installed on this box
                if rank == 0:
                    print(json.dumps({"reference": f"unavailable: {type(ex).__name__}: {ex}"}), flush=True)
        for ln in args.log2n:
            n = 1 << ln
            for d in args.density:
                eng = E.SparseAllReduce(n, None, max_density=max(0.02, d * 1.5), methods=tuple(args.plan_methods),
                                        transport=args.transport)
                x = make_inputs(n, d, P, dtype, dev, args.dist, args.overlap)[rank]
                out = torch.empty_like(x)
                def sparse():
                    eng(x, method=method, out=out)
                ref = x.clone()
                def dense():
                    dist.all_reduce(ref)
                dist.barrier()
                ms_s = time_fn(sparse, args.iters, args.warmup, flush)
                st = eng.check()
                dist.barrier()
                ms_d = time_fn(dense, args.iters, args.warmup, flush)
                want = x.clone().float(); dist.all_reduce(want)
                err = float((out.float() - want).abs().max())
                t = torch.tensor([ms_s, ms_d, float(st), err], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms_s, ms_d, stm, err = t.tolist()
                nnz = int((x != 0).sum())
                rec_bytes_out = nnz * 8 * (P - 1) / P
                em = eng.metrics()
                u = torch.tensor([float(em["union_slots"])], device=dev, dtype=torch.float64)
                dist.all_reduce(u)
                union_density = float(u.item()) / P / n                    # every rank gathers every owner's run
                ref_ms = {}
                if ref_lba is not None:
                    xr = x.clone()
                    xr[0] = 0                      # the reference cannot transmit position 0
                    for mth in (3, 2, 1):
                        try:
                            dist.barrier()
                            tm = time_fn(lambda: ref_lba.zen_sparse_comm(xr, mth), max(2, args.iters // 2), 1, flush)
                            tt = torch.tensor([tm], device=dev, dtype=torch.float64)
                            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                            ref_ms[f"reference_m{mth}_ms"] = float(tt.item())
                        except Exception as ex:
                            ref_ms[f"reference_m{mth}_ms"] = f"failed: {type(ex).__name__}"
                row = dict(mode="nvlink", transport=eng.transport, P=P, log2n=ln, density=d, dtype=args.dtype, dist=args.dist, overlap=args.overlap,
                           method=str(method), sparse_ms=ms_s, dense_nccl_ms=ms_d, speedup=ms_d / ms_s, **ref_ms,
                           eff_GBps=n * x.element_size() / ms_s / 1e6, max_err=err, status=int(stm),
                           push_bytes_per_rank=rec_bytes_out, union_density=union_density, format=em["format"][0],
                           gather_bytes_pushed=em["gather_bytes_pushed"])
                if rank == 0:
                    rows.append(row)
                    print(json.dumps(row), flush=True)
                eng.close()
                del eng, x, out, ref, want
                torch.cuda.empty_cache()
        dist.destroy_process_group()
    if args.out and rows:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")


if __name__ == "__main__":
    main()
