"""Kernel time inside real training steps (torch profiler, CUPTI kernel records; no replay, warm caches): which kernels
a step of a given model spends its time in.  One GPU, tensor parallel off, eager launches.

    python bench/step_kernel_shares.py --model llama-3-8b --micro_batch 1 --seq_len 4096 --num_layers 2
    python bench/step_kernel_shares.py --model gemma-2b --micro_batch 4 --seq_len 2048 --num_layers 2
    python bench/step_kernel_shares.py --model gpt2 --micro_batch 8 --seq_len 1024
"""
import argparse
import os
import sys

import torch
from torch.profiler import ProfilerActivity, profile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from zen_repro_b200.trainer import TrainConfig, Trainer  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--model", default="gpt2")
ap.add_argument("--micro_batch", type=int, default=8)
ap.add_argument("--seq_len", type=int, default=1024)
ap.add_argument("--num_layers", type=int, default=None)
ap.add_argument("--steps", type=int, default=2)
ap.add_argument("--top", type=int, default=24)
a = ap.parse_args()

t = Trainer(TrainConfig(model=a.model, micro_batch=a.micro_batch, seq_len=a.seq_len, num_layers=a.num_layers,
                        cuda_graph=False), init_dist=False)
ids = next(t.data)["input_ids"].to(t.device)
for _ in range(3):
    t.step_device(ids, ids)
torch.cuda.synchronize()
with profile(activities=[ProfilerActivity.CUDA]) as prof:
    for _ in range(a.steps):
        t.step_device(ids, ids)
    torch.cuda.synchronize()
rows = sorted(prof.key_averages(), key=lambda r: -r.device_time_total)
total = sum(r.device_time_total for r in rows) / a.steps
print(f"== {a.model}: {total:.0f} us of kernel time per step")
for r in rows[: a.top]:
    print(f"{r.device_time_total / a.steps:9.1f} us/step  n={r.count // a.steps:4d}  {r.key[:110]}")
