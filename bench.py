"""Headline benchmark: training throughput (tokens/s) of the flagship configuration.

    python bench.py --gpus 1 --steps 20 --warmup 5            # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W                 # N GPUs, one rank each
    python bench.py --impl reference ...                       # the reference implementation on the same config

Default config: GPT-2 small (12 layers, d 768, 12 heads, vocab 50257), bf16, data-parallel, micro-batch
8 x 1024 tokens per GPU, synthetic Zipf(1.1) tokens, random-init weights, sparse row synchronisation of
the tied token-embedding gradient and dense bucket all-reduce elsewhere.  Weak scaling (per-GPU batch
fixed).  `value` is device-timed (CUDA events around exactly K optimizer steps, max over ranks);
`e2e` times the same K steps through ``Trainer.step`` including the pinned-host -> device copy of each
batch and the device -> host read of each loss.  One JSON line is printed by rank 0.  With the default
config the line also carries ``extra``: Gemma-2B (same K and W) and GPT-2 with the framework's own top-k
hook (``--method 3 --top_k 1``, the reference arm's configuration), measured in the same process afterwards.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {
    "gpt2": dict(model="gpt2", micro_batch=8, seq_len=1024, zipf_s=1.1, tp=1),
    "gemma-2b": dict(model="gemma-2b", micro_batch=4, seq_len=2048, zipf_s=1.05, tp=1),
    "llama-3-8b": dict(model="llama-3-8b", micro_batch=1, seq_len=4096, zipf_s=1.1, tp=2),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="zen", choices=["zen", "reference"])
    ap.add_argument("--config", default="gpt2", choices=sorted(MODELS))
    ap.add_argument("--method", type=int, default=0)
    ap.add_argument("--top_k", type=float, default=1.0)
    ap.add_argument("--num_layers", type=int, default=None)
    ap.add_argument("--micro_batch", type=int, default=None)
    ap.add_argument("--no_e2e", action="store_true")
    ap.add_argument("--no_extra", action="store_true", help="skip the extra configurations measured after the GPT-2 headline")
    ap.add_argument("--bucket_cap_mb", type=float, default=None)
    ap.add_argument("--dense_transport", default=None, choices=["auto", "nccl", "nvls"],
                    help="dense buckets: library all-reduce or this library's multimem kernel through the NVSwitch")
    ap.add_argument("--no_sparse_embedding", action="store_true", help="keep the whole embedding gradient in the dense buckets")
    ap.add_argument("--no_status_mirror", action="store_true", help="do not publish the kernels' status words every step")
    ap.add_argument("--timeline", action="store_true",
                    help="after the timed passes, run K eager steps with CUDA events on the compute and communication "
                         "streams and report the communication that backward did not hide")
    ap.add_argument("--dense_embedding_under_tp", action="store_true",
                    help="TP runs: keep the vocabulary-sharded embedding gradient in the dense buckets")
    ap.add_argument("--sequence_parallel", action="store_true", help="TP layers with the residual stream sharded over tokens")
    ap.add_argument("--no_graph", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    return ap.parse_args()


def _measure(args, config_name: str, method: int, top_k: float, e2e_pass: bool) -> dict:
    """Build a ``Trainer`` for one configuration, run W warm-up steps, device-time exactly K steps (CUDA events, max over
    ranks) and, with ``e2e_pass``, time K more steps through ``Trainer.step`` from pinned host batches.  The trainer is
    torn down (graph dropped, peer regions closed) before returning, so that the next configuration starts clean."""
    import torch
    import torch.distributed as dist

    from zen_repro_b200 import _native
    from zen_repro_b200.ops import gemm
    from zen_repro_b200.trainer import TrainConfig, Trainer
    from zen_repro_b200.utils.clocks import ClockSampler

    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    preset = dict(MODELS[config_name])
    if args.micro_batch:
        preset["micro_batch"] = args.micro_batch
    if preset["tp"] > world or world % preset["tp"]:
        preset["tp"] = 1
    extra_cfg = {}
    if args.bucket_cap_mb:
        extra_cfg["bucket_cap_mb"] = args.bucket_cap_mb
    if args.dense_transport:
        extra_cfg["dense_transport"] = args.dense_transport
    if args.no_sparse_embedding:
        extra_cfg["sparse_embedding"] = False
    if args.no_status_mirror:
        extra_cfg["status_mirror"] = False
    cfg = TrainConfig(method=method, top_k=top_k, num_layers=args.num_layers, data_pool=max(4, min(8, args.steps)),
                      cuda_graph=not args.no_graph, sequence_parallel=args.sequence_parallel,
                      sparse_embedding_under_tp=preset["tp"] > 1 and not args.dense_embedding_under_tp, **extra_cfg, **preset)
    trainer = Trainer(cfg, init_dist=False)
    dev = trainer.device

    def barrier():
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    # device-resident copies of the batches for the kernel-timed region
    dev_batches = []
    for _ in range(max(4, min(8, args.steps))):
        b = next(trainer.data)
        dev_batches.append(b["input_ids"].to(dev))
    for i in range(args.warmup):
        trainer.step_device(dev_batches[i % len(dev_batches)], dev_batches[i % len(dev_batches)])
    barrier()
    sampler = ClockSampler(torch.cuda.current_device()).start() if rank == 0 else None
    l0 = _native.launch_count()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(args.steps):
        ids = dev_batches[i % len(dev_batches)]
        trainer.step_device(ids, ids)
    e.record()
    barrier()
    launches = _native.launch_count() - l0
    if trainer._graph is not None:         # replayed steps: the kernels were recorded once, at capture
        launches += trainer.graph_launches_per_step * args.steps
    ms = s.elapsed_time(e)
    # end to end through the public API: pinned host batch -> device, step, loss -> host
    e2e, e2e_ms, h2d, d2h = None, 0.0, 0, 0
    if e2e_pass:
        batches = [next(trainer.data) for _ in range(args.steps)]
        h2d, d2h = trainer.bytes_per_step(batches[0])
        barrier()
        t0 = time.perf_counter()
        for b in batches:
            trainer.step(b, read_loss=True)
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop() if sampler is not None else None
    t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    health = trainer.check_health(raise_on_error=False)
    graph_on = trainer._graph is not None                     # as the timed passes ran (the timeline below runs eagerly)
    timeline = None
    if args.timeline and world > 1:
        trainer._graph, trainer.graph_ok = None, False
        ddp_ = trainer.model.module
        ids = dev_batches[0]
        trainer.step_device(ids, ids)
        ddp_.timeline = []
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record()
        for i in range(args.steps):
            trainer.step_device(ids, ids)
        e2.record()
        rows = ddp_.exposed_comm_us()
        ddp_.timeline = None
        n_ = max(1, len(rows))
        tl = torch.tensor([sum(r["dense_exposed_us"] for r in rows) / n_, sum(r["sync_exposed_us"] for r in rows) / n_,
                           s2.elapsed_time(e2) * 1e3 / args.steps], device=dev, dtype=torch.float64)
        dist.all_reduce(tl, op=dist.ReduceOp.MAX)
        timeline = {"dense_exposed_us": tl[0].item(), "sync_exposed_us": tl[1].item(), "eager_step_us": tl[2].item(),
                    "note": "eager steps (no graph); max over ranks of the per-rank mean"}
    tokens = trainer.tokens_per_step * args.steps
    if e2e_pass:
        e2e = {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_ms / args.steps,
               "timed": "host wall clock around K calls of Trainer.step(batch): H2D copy of the pinned host batch, the "
                        "step, loss.item(); a separate pass over fresh batches, after the device-timed pass"}
    ddp = trainer.model.module
    out = {
        "metric": "train tokens/sec", "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic Zipf tokens, random-init weights", "impl": "zen",
        "config": {"model": cfg.model, "global_batch": cfg.micro_batch * trainer.plugin.dp_size, "seq_len": cfg.seq_len,
                   "parallelism": f"dp{trainer.plugin.dp_size}" + (f"xtp{cfg.tp}" if cfg.tp > 1 else "") + ("+sp" if (cfg.tp > 1 and cfg.sequence_parallel) else ""),
                   "method": cfg.method, "top_k": cfg.top_k,
                   # what was actually built, not what was asked for
                   "embedding_row_sync": ddp.embedding_sync is not None, "bucket_cap_mb": cfg.bucket_cap_mb,
                   "n_buckets": len(ddp.buckets), "dense_allreduce": "nvls multimem kernel" if getattr(ddp, "arena", None) is not None else "nccl", "grad_checkpoint": bool(trainer.model_cfg.grad_checkpoint),
                   "num_layers": trainer.model_cfg.num_layers, "cuda_graph": bool(graph_on),
                   "weight_grad_group": int(gemm.GROUP_SIZE),
                   "l2": "per-step working set (weights + activations, > 1 GB) exceeds the 126 MB L2"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "gemm_error": gemm.gemm_error(),
        "kernel_status": {k: v for k, v in health.items() if v},
    }
    if timeline is not None:
        out["timeline"] = timeline
    trainer.close()
    del trainer, dev_batches
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    return out


def run_zen(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or "RANK" in os.environ:
        from zen_repro_b200.parallel import launch_from_torch

        launch_from_torch()
    rank = dist.get_rank() if dist.is_initialized() else 0
    try:
        out = _measure(args, args.config, args.method, args.top_k, not args.no_e2e)
    except Exception as ex:
        if args.dense_transport not in (None, "auto"):
            raise
        # the multicast path for the dense buckets is the one piece that depends on the fabric: measure on NCCL instead
        import traceback

        traceback.print_exc()
        args.dense_transport = "nccl"
        out = _measure(args, args.config, args.method, args.top_k, not args.no_e2e)
        out["note"] = f"dense buckets fell back to NCCL after {type(ex).__name__}"
    if args.config == "gpt2" and args.method == 0 and not args.no_extra:
        # measured in the same process after the headline, same K and W: the second model of the benchmark, and the
        # framework's own top-k hook in the reference arm's configuration (method 3, top_k 1; train.py:99-100)
        extra = {}
        for name, (cfg_name, method, top_k) in {"gemma-2b": ("gemma-2b", 0, 1.0), "gpt2_method3": ("gpt2", 3, 1.0)}.items():
            try:
                r = _measure(args, cfg_name, method, top_k, True)
                extra[name] = {k: r[k] for k in ("value", "unit", "ms_per_step", "config", "e2e", "gpu_launches", "kernel_status")}
            except Exception as ex:  # a failed extra must not cost the headline
                extra[name] = {"error": f"{type(ex).__name__}: {ex}"[:300]}
        out["extra"] = extra
    if rank == 0:
        print(json.dumps(out), flush=True)
    if dist.is_initialized():
        dist.barrier()
        torch.cuda.synchronize()
        dist.destroy_process_group()


def main():
    args = parse()
    try:
        if args.impl == "reference":
            from baseline.reference_arm import run_reference

            run_reference(args, MODELS[args.config], MODELS)
        else:
            run_zen(args)
    except SystemExit:
        raise
    except BaseException:
        # leave at once: a rank that lingers in teardown after an error keeps its peers waiting in a collective
        import traceback

        traceback.print_exc()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(1)


if __name__ == "__main__":
    main()
