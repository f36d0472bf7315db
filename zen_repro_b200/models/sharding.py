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
