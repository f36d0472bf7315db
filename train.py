"""Training entry point with the reference's flags (train.py:91-105) and result sinks.

    torchrun --nproc-per-node 8 train.py --model_name gpt2 --tp 1 --method 0 -b 8 -l 1024
    torchrun --nproc-per-node 8 train.py --model_name meta-llama/Llama-3.2-3B --tp 2 --method 3 --top_k 1

``--method`` 0 = dense bucket all-reduce (mean) with the token-embedding gradient synchronised as sparse rows;
1 / 2 / 3 = the ZEN hook on every bucket (sampled top-k, then sparse all-gather / balanced exchange with COO /
balanced exchange with bitmap; SUM over data-parallel ranks).  As in the reference, steps 80..95 are timed and
``time.txt`` receives ``"{model} method {m} topk {k} dp {P}"`` and the seconds per iteration; here the interval
is measured with CUDA events (max over ranks) and also written as JSON lines to ``--metrics_out``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from zen_repro_b200.ckpt import load_checkpoint, save_checkpoint  # noqa: E402
from zen_repro_b200.parallel import launch_from_torch  # noqa: E402
from zen_repro_b200.trainer import TrainConfig, Trainer  # noqa: E402
from zen_repro_b200.utils import set_seed, setup_logger, trace_range  # noqa: E402


def build_parser():
    p = argparse.ArgumentParser()
    p.add_argument("--model_name", type=str, default="facebook/opt-2.7b", help="Model name")
    p.add_argument("-b", "--batch_size", type=int, default=1, help="Batch size")
    p.add_argument("-s", "--num_steps", type=int, default=100, help="Number of steps to run")
    p.add_argument("-g", "--grad_checkpoint", action="store_true", default=True, help="Enable gradient checkpointing")
    p.add_argument("--no_grad_checkpoint", dest="grad_checkpoint", action="store_false")
    p.add_argument("-l", "--max_length", type=int, default=1024, help="Max sequence length")
    p.add_argument("--tp", type=int, default=2, help="Tensor parallel size")
    p.add_argument("--top_k", type=int, default=1, help="Top-k percent kept by the sparsifier")
    p.add_argument("--seed", type=int, default=0, help="Random seed")
    p.add_argument("--method", type=int, default=3, help="0 dense, 1 sparse all-gather, 2 ZEN (COO), 3 ZEN (bitmap)")
    p.add_argument("--bucket_cap", type=int, default=512, help="Bucket cap in MB")
    p.add_argument("--num_hidden_layers", type=int, default=None)
    p.add_argument("--kv_heads", type=int, default=None)
    # additions
    p.add_argument("--data", choices=["synthetic", "hf"], default="synthetic")
    p.add_argument("--zipf_s", type=float, default=1.1)
    p.add_argument("--no_sparse_embedding", action="store_true")
    p.add_argument("--sequence_parallel", action="store_true", help="TP with the residual stream sharded over tokens")
    p.add_argument("--save", type=str, default=None, help="checkpoint directory written at the end")
    p.add_argument("--resume", type=str, default=None, help="checkpoint directory to resume from")
    p.add_argument("--metrics_out", type=str, default=None, help="JSON-lines file: per-step records and the final summary")
    p.add_argument("--metrics_every", type=int, default=0,
                   help="> 0: every N-th step also collect the counters of the sparse paths (one device synchronisation)")
    p.add_argument("--profile_steps", type=int, default=0,
                   help="> 0: after the run, record this many more steps with the torch profiler and print the kernels that "
                        "the step spends its device time in (launches come from the host for these steps)")
    p.add_argument("--trace", action="store_true", help="NVTX ranges with the reference's names around every stage")
    p.add_argument("--log_dir", type=str, default=".")
    p.add_argument("--time_file", type=str, default="time.txt", help="the reference's result sink (appended to)")
    p.add_argument("--time_from", type=int, default=80)
    p.add_argument("--time_to", type=int, default=95)
    return p


def kernel_shares(trainer, steps: int, coord, top: int = 24) -> None:
    """Kernel time inside real training steps (torch profiler, CUPTI kernel records: no replay, warm caches)."""
    from torch.profiler import ProfilerActivity, profile

    trainer._graph, trainer.graph_ok = None, False
    ids = next(trainer.data)["input_ids"].to(trainer.device)
    trainer.step_device(ids, ids)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            trainer.step_device(ids, ids)
        torch.cuda.synchronize()
    rows = sorted(prof.key_averages(), key=lambda r: -r.device_time_total)
    total = sum(r.device_time_total for r in rows) / steps
    coord.print_on_master(f"== {trainer.cfg.model}: {total:.0f} us of kernel time per step")
    for r in rows[:top]:
        coord.print_on_master(f"{r.device_time_total / steps:9.1f} us/step  n={r.count // steps:4d}  {r.key[:110]}")


def main(argv=None):
    args = build_parser().parse_args(argv)
    set_seed(args.seed)
    if args.trace:
        from zen_repro_b200.utils import enable_tracing

        enable_tracing(True)
    rank, world, device = launch_from_torch()
    logger = setup_logger(args.log_dir)
    tp = args.tp if world % args.tp == 0 and args.tp <= world else 1
    cfg = TrainConfig(model=args.model_name, micro_batch=args.batch_size, seq_len=args.max_length, tp=tp,
                      method=args.method, top_k=args.top_k, bucket_cap_mb=args.bucket_cap,
                      sparse_embedding=not args.no_sparse_embedding, grad_checkpoint=args.grad_checkpoint,
                      zipf_s=args.zipf_s, seed=args.seed, num_layers=args.num_hidden_layers, kv_heads=args.kv_heads,
                      data_pool=0, sequence_parallel=args.sequence_parallel)
    trainer = Trainer(cfg, init_dist=False)
    coord = trainer.coordinator
    if args.data == "hf":
        from zen_repro_b200.data.hf import hf_token_stream

        trainer.data = hf_token_stream(args.model_name, args.max_length, args.batch_size, trainer.plugin, args.seed)
    if args.resume:
        logger.info(f"resumed from {args.resume} at step {load_checkpoint(args.resume, trainer)}")
    mem = torch.cuda.max_memory_allocated() / 1024 ** 2 if torch.cuda.is_available() else 0.0
    coord.print_on_master(f"Booster init max CUDA memory: {mem:.2f} MB")
    t_from, t_to = args.time_from, min(args.time_to, args.num_steps)
    ev0 = ev1 = None
    wall0 = wall1 = None
    for step in range(args.num_steps + 1):
        if step == t_from:
            wall0 = time.time()
            if device.type == "cuda":
                ev0 = torch.cuda.Event(enable_timing=True); ev0.record()
        if step == t_to:
            wall1 = time.time()
            if device.type == "cuda":
                ev1 = torch.cuda.Event(enable_timing=True); ev1.record()
        batch = next(trainer.data)
        t_step = time.perf_counter()
        loss = trainer.step(batch, read_loss=True)
        step_ms = (time.perf_counter() - t_step) * 1e3
        coord.print_on_master(f"Step {step} loss: {loss}")
        if args.metrics_out:
            rec = {"kind": "step", "step": step, "loss": loss, "step_ms": step_ms}
            if args.metrics_every > 0 and step % args.metrics_every == 0:
                rec.update(trainer.collect_metrics())
            if coord.is_master():
                with open(args.metrics_out, "a") as f:
                    f.write(json.dumps(rec) + "\n")
        if step >= args.num_steps:
            break
    mem = torch.cuda.max_memory_allocated() / 1024 ** 2 if torch.cuda.is_available() else 0.0
    coord.print_on_master(f"Max CUDA memory usage: {mem:.2f} MB")
    health = trainer.check_health(raise_on_error=False)          # status words of the kernels (0 = clean)
    if any(health.values()):
        print(f"[rank {dist.get_rank() if dist.is_initialized() else 0}] kernel status: {health}", flush=True)
    dp = trainer.plugin.dp_size
    header = f"{args.model_name} method {args.method} topk {args.top_k} dp {dp}"
    sec_per_it = None
    if wall0 is not None and wall1 is not None and t_to > t_from:
        if ev0 is not None:
            torch.cuda.synchronize()
            t = torch.tensor([ev0.elapsed_time(ev1) / 1e3], device=device, dtype=torch.float64)
            if dist.is_initialized() and world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec_per_it = float(t.item()) / (t_to - t_from)
        else:
            sec_per_it = (wall1 - wall0) / (t_to - t_from)
    coord.print_on_master(header + "\n")
    coord.print_on_master(f"{sec_per_it}\n")
    if coord.is_master():
        with open(args.time_file, "a") as f:
            f.write(header + "\n")
            f.write(f"{sec_per_it}\n")
        if args.metrics_out and sec_per_it:
            with open(args.metrics_out, "a") as f:
                f.write(json.dumps({"kind": "summary", "model": args.model_name, "method": args.method, "top_k": args.top_k, "dp": dp, "tp": tp,
                                    "sec_per_iter": sec_per_it, "tokens_per_s": trainer.tokens_per_step / sec_per_it,
                                    "max_mem_mb": mem, "recoveries": trainer.recoveries, "kernel_status": health,
                                    "config": cfg.to_dict()}) + "\n")
    if args.profile_steps > 0 and device.type == "cuda":
        kernel_shares(trainer, args.profile_steps, coord)
    if args.save:
        save_checkpoint(args.save, trainer)
    trainer.close()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
