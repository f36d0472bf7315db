"""Sparsity / skew analysis with CSV sinks (capability of the reference's ``Logger``, utils.py:40-150).

Files go under ``results/{model}_{partition}/batchsize_{b}_top_k_{k}_{kind}.csv``.  ``log_skewness``
thresholds a gradient at its exact top-k, splits it into ``partition`` contiguous parts along its
longer axis and records each part's share of the surviving entries; the distributed form samples the
threshold and reduces over ranks; ``log_sparsity`` records per-parameter zero fractions.
"""
from __future__ import annotations

import csv
import math
import os

import torch
import torch.distributed as dist


def calculate_sparsity(t: torch.Tensor) -> float:
    """Fraction of exact zeros."""
    n = t.numel()
    return float((t == 0).sum().item()) / n if n else 0.0


def exact_topk_threshold(t: torch.Tensor, top_k_percent: float) -> torch.Tensor:
    flat = t.detach().abs().reshape(-1).float()
    k = max(1, int(flat.numel() * top_k_percent / 100))
    return torch.topk(flat, k, sorted=False)[0].min()


def sampled_topk_threshold(t: torch.Tensor, top_k_percent: float, group=None, sample_frac: float = 0.01,
                           generator=None) -> torch.Tensor:
    """Threshold from a random sample of |t| (with replacement), all-gathered over ``group`` when given."""
    flat = t.detach().abs().reshape(-1)
    n = flat.numel()
    ns = max(1, math.ceil(sample_frac * n))
    pos = torch.randint(0, n, (ns,), device=flat.device, generator=generator)
    sample = flat[pos]
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        out = torch.empty(dist.get_world_size(group) * ns, dtype=sample.dtype, device=sample.device)
        dist.all_gather_into_tensor(out, sample.contiguous(), group=group)
        sample = out
    k = max(1, sample.numel() * int(top_k_percent) // 100) if float(top_k_percent).is_integer() else \
        max(1, int(sample.numel() * top_k_percent / 100))
    return torch.topk(sample.float(), k, sorted=False)[0].min()


def partition_shares(mask: torch.Tensor, partition: int) -> list[float]:
    """Share of nonzeros in each of ``partition`` contiguous chunks along the longer axis."""
    m = mask if mask.dim() > 1 else mask.reshape(1, -1)
    axis = 0 if m.shape[0] >= m.shape[-1] else m.dim() - 1
    chunks = torch.chunk(m, partition, dim=axis)
    total = max(1, int(mask.sum().item()))
    return [float(c.sum().item()) / total for c in chunks]


class SparsityLogger:
    def __init__(self, model_name: str, partition: int, batch_size: int, top_k: float, root: str = "results"):
        self.partition, self.top_k = partition, top_k
        self.dir = os.path.join(root, f"{model_name.replace('/', '_')}_{partition}")
        self.prefix = f"batchsize_{batch_size}_top_k_{top_k}"

    def _write(self, kind: str, row: list):
        os.makedirs(self.dir, exist_ok=True)
        with open(os.path.join(self.dir, f"{self.prefix}_{kind}.csv"), "a", newline="") as f:
            csv.writer(f).writerow(row)

    def log_skewness(self, name: str, grad: torch.Tensor, step: int = 0):
        thr = exact_topk_threshold(grad, self.top_k)
        mask = grad.detach().abs() >= thr
        shares = partition_shares(mask, self.partition)
        self._write("skewness", [step, name, int(mask.sum())] + shares)
        return shares

    def log_skewness_distributed(self, name: str, grad: torch.Tensor, step: int = 0, group=None):
        thr = sampled_topk_threshold(grad, self.top_k, group)
        mask = grad.detach().abs() >= thr
        shares = torch.tensor(partition_shares(mask, self.partition), device=grad.device)
        count = mask.sum().reshape(1).float()
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            P = dist.get_world_size(group)
            counts = torch.empty(P, device=grad.device)
            all_sh = torch.empty(P * self.partition, device=grad.device)
            dist.all_gather_into_tensor(counts, count, group=group)
            dist.all_gather_into_tensor(all_sh, shares, group=group)
            if dist.get_rank(group) == 0:
                self._write("skewness_distributed", [step, name] + counts.tolist() + all_sh.tolist())
        else:
            self._write("skewness_distributed", [step, name, float(count)] + shares.tolist())
        return shares.tolist()

    def log_sparsity(self, model: torch.nn.Module, step: int = 0, apply_threshold: bool = False):
        """Per-parameter zero fraction of the gradients; optionally replaces each gradient by its thresholded form."""
        out = {}
        for n, p in model.named_parameters():
            if p.grad is None:
                continue
            g = p.grad
            if apply_threshold and g.numel() > 4096:
                thr = exact_topk_threshold(g, self.top_k)
                g = torch.where(g.abs() >= thr, g, torch.zeros_like(g))
                p.grad = g
            out[n] = calculate_sparsity(g)
            self._write("sparsity", [step, n, out[n]])
        return out
