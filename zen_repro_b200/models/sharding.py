"""Tensor-parallel sharding of a full (TP = 1) native state dict, and the inverse gather.

Column-parallel matrices (qkv, gate|up) are split along their output dimension head by head / half by
half so that every rank holds whole heads and matching gate and up slices; row-parallel matrices
(attention out, down) along their input dimension; embeddings and the LM head along the (padded)
vocabulary; norms and row-parallel biases are replicated.  This is the sharding ColossalAI's shardformer
policies apply for the reference (train.py:117-123).
"""
from __future__ import annotations

import torch

from .config import ModelConfig


def _out_slice(w, sl, layout):
    return w[:, sl] if layout == "in_out" else w[sl]


def _in_slice(w, sl, layout):
    return w[sl] if layout == "in_out" else w[:, sl]


def shard_state_dict(full: dict, cfg: ModelConfig, tp_rank: int, tp: int) -> dict:
    if tp == 1:
        return dict(full)
    hd, lay = cfg.head_dim, cfg.weight_layout
    hq_l = cfg.num_heads // tp
    kv_rep = cfg.num_kv_heads < tp
    hkv_l = 1 if kv_rep else cfg.num_kv_heads // tp
    I_l = cfg.intermediate_size // tp
    qs, ks = cfg.num_heads * hd, cfg.num_kv_heads * hd
    out = {}

    def qkv_index():
        q = torch.arange(tp_rank * hq_l * hd, (tp_rank + 1) * hq_l * hd)
        kv_head0 = (tp_rank * cfg.num_kv_heads // tp) if kv_rep else tp_rank * hkv_l
        k = qs + torch.arange(kv_head0 * hd, (kv_head0 + hkv_l) * hd)
        v = qs + ks + torch.arange(kv_head0 * hd, (kv_head0 + hkv_l) * hd)
        return torch.cat([q, k, v])

    def up_index():
        base = torch.arange(tp_rank * I_l, (tp_rank + 1) * I_l)
        return torch.cat([base, cfg.intermediate_size + base]) if cfg.gated else base

    qi, ui = qkv_index(), up_index()
    vpad = (cfg.vocab_size + tp - 1) // tp * tp
    vl = vpad // tp
    for k, v in full.items():
        name = k.split(".")[-1]
        if name == "qkv_w":
            out[k] = _out_slice(v, qi, lay).clone()
        elif name == "qkv_b":
            out[k] = v[qi].clone()
        elif name == "up_w":
            out[k] = _out_slice(v, ui, lay).clone()
        elif name == "up_b":
            out[k] = v[ui].clone()
        elif name == "o_w":
            out[k] = _in_slice(v, slice(tp_rank * hq_l * hd, (tp_rank + 1) * hq_l * hd), lay).clone()
        elif name == "down_w":
            out[k] = _in_slice(v, slice(tp_rank * I_l, (tp_rank + 1) * I_l), lay).clone()
        elif name in ("wte", "lm_head"):
            padded = torch.zeros(vpad, v.shape[1], dtype=v.dtype)
            padded[: v.shape[0]] = v
            out[k] = padded[tp_rank * vl:(tp_rank + 1) * vl].clone()
        else:
            out[k] = v.clone()
    return out


def _index_sets(cfg: ModelConfig, tp_rank: int, tp: int):
    """Row indices of the fused qkv and gate|up outputs held by ``tp_rank`` (the same sets shard_state_dict cuts)."""
    hd = cfg.head_dim
    hq_l = cfg.num_heads // tp
    kv_rep = cfg.num_kv_heads < tp
    hkv_l = 1 if kv_rep else cfg.num_kv_heads // tp
    I_l = cfg.intermediate_size // tp
    qs, ks = cfg.num_heads * hd, cfg.num_kv_heads * hd
    q = torch.arange(tp_rank * hq_l * hd, (tp_rank + 1) * hq_l * hd)
    kv_head0 = (tp_rank * cfg.num_kv_heads // tp) if kv_rep else tp_rank * hkv_l
    k = qs + torch.arange(kv_head0 * hd, (kv_head0 + hkv_l) * hd)
    v = qs + ks + torch.arange(kv_head0 * hd, (kv_head0 + hkv_l) * hd)
    base = torch.arange(tp_rank * I_l, (tp_rank + 1) * I_l)
    up = torch.cat([base, cfg.intermediate_size + base]) if cfg.gated else base
    return torch.cat([q, k, v]), up


def unshard_state_dicts(shards: list, cfg: ModelConfig) -> dict:
    """Inverse of ``shard_state_dict``: the TP shards (rank order) of a native state dict, or of any per-parameter
    state with the parameters' shapes (optimizer moments, master weights), joined into the full TP = 1 form.
    Replicated entries are taken from rank 0; a KV head replicated over several ranks likewise from the first holder."""
    tp = len(shards)
    if tp == 1:
        return dict(shards[0])
    hd, lay = cfg.head_dim, cfg.weight_layout
    qkv_rows = (cfg.num_heads + 2 * cfg.num_kv_heads) * hd
    up_rows = cfg.intermediate_size * (2 if cfg.gated else 1)
    idx = [_index_sets(cfg, r, tp) for r in range(tp)]
    out = {}
    for k, v0 in shards[0].items():
        name = k.split(".")[-1]
        parts = [sh[k] for sh in shards]
        if name in ("qkv_w", "qkv_b", "up_w", "up_b"):
            rows = qkv_rows if name.startswith("qkv") else up_rows
            which = 0 if name.startswith("qkv") else 1
            if name.endswith("_b"):
                full = torch.zeros(rows, dtype=v0.dtype)
                for r in reversed(range(tp)):               # lower ranks win where a KV head is replicated
                    full[idx[r][which]] = parts[r]
            elif lay == "in_out":
                full = torch.zeros(v0.shape[0], rows, dtype=v0.dtype)
                for r in reversed(range(tp)):
                    full[:, idx[r][which]] = parts[r]
            else:
                full = torch.zeros(rows, v0.shape[1], dtype=v0.dtype)
                for r in reversed(range(tp)):
                    full[idx[r][which]] = parts[r]
            out[k] = full
        elif name in ("o_w", "down_w"):
            out[k] = torch.cat(parts, dim=0 if lay == "in_out" else 1)
        elif name in ("wte", "lm_head"):
            out[k] = torch.cat(parts, dim=0)[: cfg.vocab_size].clone()
        else:
            out[k] = v0.clone()
    return out
