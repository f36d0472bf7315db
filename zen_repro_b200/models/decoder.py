"""Decoder-only language model on the framework's own ops.

One implementation serves GPT-2, OPT, Llama and Gemma; ``ModelConfig`` selects norms, activations,
positions, weight layout and biases.  Projections are stored fused (one qkv matrix, one gate|up
matrix) because one wide GEMM beats three narrow ones; ``hf_state_dict`` / ``load_hf_state_dict``
split and join them so that checkpoints carry HuggingFace parameter names and shapes.

Pre-norm blocks; the residual add is fused into the following norm kernel, so a block passes on
(branch output, residual stream) rather than their sum.  Tensor parallelism is Megatron-style 1-D:
qkv / gate|up are column-parallel, attention-out / down are row-parallel, embeddings and the LM head
are vocab-parallel.  The reference obtains models from ``AutoModelForCausalLM.from_config`` and
tensor parallelism from ColossalAI's shardformer (train.py:117-123, 149-157).
"""
from __future__ import annotations


import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..ops import autograd as O
from .config import ModelConfig


def _tp(group) -> tuple[int, int]:
    if group is None:
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


class Block(nn.Module):
    def __init__(self, cfg: ModelConfig, tp_group=None, device=None, dtype=None):
        super().__init__()
        self.cfg, self.tp_group = cfg, tp_group
        _, tp = _tp(tp_group)
        d, hd = cfg.hidden_size, cfg.head_dim
        assert cfg.num_heads % tp == 0 and (cfg.num_kv_heads % tp == 0 or cfg.num_kv_heads < tp)
        self.hq = cfg.num_heads // tp
        self.hkv = max(1, cfg.num_kv_heads // tp)         # MQA under TP replicates the single KV head
        self.kv_replicated = cfg.num_kv_heads < tp
        self.inner = cfg.intermediate_size // tp
        kw = dict(device=device, dtype=dtype)
        qkv_out = (self.hq + 2 * self.hkv) * hd
        up_out = self.inner * (2 if cfg.gated else 1)

        def w(i, o):
            return nn.Parameter(torch.empty((i, o) if cfg.weight_layout == "in_out" else (o, i), **kw))

        self.norm1_w = nn.Parameter(torch.empty(d, **kw))
        self.norm2_w = nn.Parameter(torch.empty(d, **kw))
        # Gemma-2: a second norm on the output of each branch, before it joins the residual stream
        self.postnorm1_w = nn.Parameter(torch.empty(d, **kw)) if cfg.post_norms else None
        self.postnorm2_w = nn.Parameter(torch.empty(d, **kw)) if cfg.post_norms else None
        self.qkv_w, self.o_w = w(d, qkv_out), w(self.hq * hd, d)
        self.up_w, self.down_w = w(d, up_out), w(self.inner, d)
        if cfg.has_bias:
            self.norm1_b = nn.Parameter(torch.empty(d, **kw))
            self.norm2_b = nn.Parameter(torch.empty(d, **kw))
            self.qkv_b = nn.Parameter(torch.empty(qkv_out, **kw))
            self.o_b = nn.Parameter(torch.empty(d, **kw))
            self.up_b = nn.Parameter(torch.empty(up_out, **kw))
            self.down_b = nn.Parameter(torch.empty(d, **kw))
        else:
            self.norm1_b = self.norm2_b = self.qkv_b = self.o_b = self.up_b = self.down_b = None

    def _post(self, x, w):
        """Branch-output norm of Gemma-2 (identity for the other families)."""
        if w is None:
            return x
        cfg = self.cfg
        return O.fused_norm(x, None, w, None, cfg.norm_eps, cfg.layer_norm, cfg.norm_unit_offset)[0]

    def _attend(self, qkv, bsz, seq):
        cfg = self.cfg
        if cfg.sliding_window and seq > cfg.sliding_window:
            raise NotImplementedError(f"sequence length {seq} exceeds the sliding window {cfg.sliding_window}: windowed "
                                      f"attention layers are only run where the window covers the whole sequence")
        return O.attention(qkv, bsz, seq, self.hq, self.hkv, cfg.head_dim, softcap=cfg.attn_softcap)

    tp_ws = None        # FusedTPWorkspace shared by all blocks of a model (set by DecoderLM.enable_fused_tp)
    sequence_parallel = False   # residual stream sharded over the tokens of the TP group (DecoderLM.enable_sequence_parallel)

    def forward(self, x, res, bsz: int, seq: int):
        cfg, g = self.cfg, self.tp_group
        rank, tp = _tp(g)
        if self.sequence_parallel and tp > 1:
            return self._forward_sp(x, res, bsz, seq)
        ws = self.tp_ws if (tp > 1 and x.is_cuda and x.dtype == torch.bfloat16) else None
        if ws is not None and ws.fits(x.shape[0], cfg.hidden_size):
            return self._forward_fused_tp(x, res, bsz, seq, ws)
        y, h = O.fused_norm(x, res, self.norm1_w, self.norm1_b, cfg.norm_eps, cfg.layer_norm, cfg.norm_unit_offset)
        y = O.copy_to_tp(y, g)
        qkv = O.linear(y, self.qkv_w, self.qkv_b, cfg.weight_layout)
        if not cfg.learned_positions:
            qkv = O.rope_qkv(qkv, self.hq, self.hkv, cfg.head_dim, seq, cfg.rope_theta)
        a = self._attend(qkv, bsz, seq)
        # the bias of a row-parallel layer is added once, after the reduction
        o = O.linear(a, self.o_w, self.o_b if tp == 1 else None, cfg.weight_layout)
        o = O.reduce_from_tp(o, g)
        if tp > 1 and self.o_b is not None:
            o = o + self.o_b
        o = self._post(o, self.postnorm1_w)
        y2, h2 = O.fused_norm(o, h, self.norm2_w, self.norm2_b, cfg.norm_eps, cfg.layer_norm, cfg.norm_unit_offset)
        y2 = O.copy_to_tp(y2, g)
        u = O.linear(y2, self.up_w, self.up_b, cfg.weight_layout)
        m = O.activation(u, cfg.act)
        dn = O.linear(m, self.down_w, self.down_b if tp == 1 else None, cfg.weight_layout)
        dn = O.reduce_from_tp(dn, g)
        if tp > 1 and self.down_b is not None:
            dn = dn + self.down_b
        return self._post(dn, self.postnorm2_w), h2


def _block_forward_fused_tp(self, x, res, bsz, seq, ws):
    """Tensor-parallel block with both all-reduces of the forward (attention out, MLP down) and both of the backward
    (qkv and up input gradients) fused into the GEMM epilogues."""
    cfg = self.cfg
    y, h = O.fused_norm(x, res, self.norm1_w, self.norm1_b, cfg.norm_eps, cfg.layer_norm, cfg.norm_unit_offset)
    qkv = O.linear(y, self.qkv_w, self.qkv_b, cfg.weight_layout, "col", ws)
    if not cfg.learned_positions:
        qkv = O.rope_qkv(qkv, self.hq, self.hkv, cfg.head_dim, seq, cfg.rope_theta)
    a = self._attend(qkv, bsz, seq)
    o = self._post(O.linear(a, self.o_w, self.o_b, cfg.weight_layout, "row", ws), self.postnorm1_w)
    y2, h2 = O.fused_norm(o, h, self.norm2_w, self.norm2_b, cfg.norm_eps, cfg.layer_norm, cfg.norm_unit_offset)
    u = O.linear(y2, self.up_w, self.up_b, cfg.weight_layout, "col", ws)
    m = O.activation(u, cfg.act)
    dn = O.linear(m, self.down_w, self.down_b, cfg.weight_layout, "row", ws)
    return self._post(dn, self.postnorm2_w), h2


Block._forward_fused_tp = _block_forward_fused_tp


def _block_forward_sp(self, x, res, bsz, seq):
    """Sequence-parallel block: x and res hold this rank's T / P token rows.  Norms run on the shard; the
    column-parallel projections gather the tokens inside the GEMM (all-gather + GEMM), attention and the activation see
    all tokens and this rank's heads / inner columns; the row-parallel projections return this rank's rows of the sum
    (GEMM + reduce-scatter).  The reference's ColossalAI plugin has this mode too (enable_sequence_parallelism) but
    train.py:117-123 leaves it off."""
    cfg, g = self.cfg, self.tp_group
    ws = self.tp_ws if (x.is_cuda and x.dtype == torch.bfloat16) else None
    lay = cfg.weight_layout
    y, h = O.fused_norm(x, res, self.norm1_w, self.norm1_b, cfg.norm_eps, cfg.layer_norm, cfg.norm_unit_offset)
    qkv = O.sp_linear(y, self.qkv_w, self.qkv_b, lay, "ag", g, ws)
    if not cfg.learned_positions:
        qkv = O.rope_qkv(qkv, self.hq, self.hkv, cfg.head_dim, seq, cfg.rope_theta)
    a = self._attend(qkv, bsz, seq)
    o = self._post(O.sp_linear(a, self.o_w, self.o_b, lay, "rs", g, ws), self.postnorm1_w)
    y2, h2 = O.fused_norm(o, h, self.norm2_w, self.norm2_b, cfg.norm_eps, cfg.layer_norm, cfg.norm_unit_offset)
    u = O.sp_linear(y2, self.up_w, self.up_b, lay, "ag", g, ws)
    m = O.activation(u, cfg.act)
    dn = O.sp_linear(m, self.down_w, self.down_b, lay, "rs", g, ws)
    return self._post(dn, self.postnorm2_w), h2


Block._forward_sp = _block_forward_sp


class DecoderLM(nn.Module):
    """Causal LM.  ``forward(input_ids, labels)`` returns the mean next-token loss."""

    def __init__(self, cfg: ModelConfig, tp_group=None, device=None, dtype=torch.bfloat16, sparse_sink=None):
        super().__init__()
        self.cfg, self.tp_group = cfg, tp_group
        rank, tp = _tp(tp_group)
        kw = dict(device=device, dtype=dtype)
        d = cfg.hidden_size
        self.vocab_padded = (cfg.vocab_size + tp - 1) // tp * tp
        self.vocab_local = self.vocab_padded // tp
        self.vocab_start = rank * self.vocab_local
        self.wte = nn.Parameter(torch.empty(self.vocab_local, d, **kw))
        self.wpe = nn.Parameter(torch.empty(cfg.max_position + cfg.pos_offset, d, **kw)) if cfg.learned_positions else None
        self.blocks = nn.ModuleList([Block(cfg, tp_group, device, dtype) for _ in range(cfg.num_layers)])
        self.norm_f_w = nn.Parameter(torch.empty(d, **kw))
        self.norm_f_b = nn.Parameter(torch.empty(d, **kw)) if cfg.has_bias else None
        self.lm_head = None if cfg.tie_embeddings else nn.Parameter(torch.empty(self.vocab_local, d, **kw))
        self.sparse_sink = sparse_sink          # receives the row-sparse lookup gradient of wte when set
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self, seed: int | None = None):
        cfg = self.cfg
        gen = None
        if seed is not None:
            gen = torch.Generator(device=self.wte.device).manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith("_b"):
                p.zero_()
            elif "norm" in name:
                p.fill_(0.0 if cfg.norm_unit_offset else 1.0)
            else:
                p.normal_(0.0, cfg.init_std, generator=gen)

    def enable_fused_tp(self, max_tokens: int, backend: str | None = None):
        """Allocate the symmetric exchange workspace (collective over the TP group) and switch the blocks to the
        GEMMs with the all-reduce fused into their epilogue."""
        from ..parallel.tp_fused import FusedTPWorkspace

        _, tp = _tp(self.tp_group)
        if tp > 1 and self.wte.is_cuda:
            ws = FusedTPWorkspace(self.tp_group, max_tokens, self.cfg.hidden_size, backend=backend)
            for b in self.blocks:
                b.tp_ws = ws
            self.tp_ws = ws
        return self

    def disable_fused_tp(self):
        """Back to GEMM + NCCL all-reduce for the tensor-parallel layers (the workspace stays allocated)."""
        for b in self.blocks:
            b.tp_ws = None
        self._tp_ws_off, self.tp_ws = getattr(self, "tp_ws", None), None
        return self

    def enable_sequence_parallel(self, on: bool = True):
        """Shard the residual stream over the tokens of the TP group (tokens per step must divide by the group size).
        Norm parameters and the biases of row-parallel layers then see only this rank's tokens; their gradients are
        summed over the group by ``sync_replicated_grads``."""
        _, tp = _tp(self.tp_group)
        self.sequence_parallel = bool(on) and tp > 1
        for b in self.blocks:
            b.sequence_parallel = self.sequence_parallel
        return self

    def _sp_partial_params(self):
        ps = [self.norm_f_w, self.norm_f_b]
        for b in self.blocks:
            ps += [b.norm1_w, b.norm2_w, b.norm1_b, b.norm2_b, b.o_b, b.down_b, b.postnorm1_w, b.postnorm2_w]
        return [p for p in ps if p is not None]

    def head_weight(self):
        return self.wte if self.lm_head is None else self.lm_head

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None, shift_labels: bool = True):
        cfg = self.cfg
        bsz, seq = input_ids.shape
        _, tp = _tp(self.tp_group)
        ids = input_ids.reshape(-1)
        if tp > 1:
            x = self._vocab_parallel_embed(ids, seq)
        else:
            x = O.embedding(ids, self.wte, self.wpe, seq, cfg.pos_offset, cfg.embed_scale, self.sparse_sink)
        res = None
        sp = getattr(self, "sequence_parallel", False) and tp > 1
        if sp:
            assert ids.numel() % tp == 0, "sequence parallelism needs the token count to divide by the TP size"
            x = O.scatter_to_sp(x, self.tp_group)
        for blk in self.blocks:
            if cfg.grad_checkpoint and torch.is_grad_enabled():
                x, res = checkpoint(blk, x, res, bsz, seq, use_reentrant=False)
            else:
                x, res = blk(x, res, bsz, seq)
        y, _ = O.fused_norm(x, res, self.norm_f_w, self.norm_f_b, cfg.norm_eps, cfg.layer_norm, cfg.norm_unit_offset)
        if sp:
            y = O.gather_from_sp(y, self.tp_group)
        if labels is None:
            logits = self._logits(y).view(bsz, seq, -1)
            if cfg.final_softcap > 0:
                logits = cfg.final_softcap * torch.tanh(logits.float() / cfg.final_softcap)
            return logits
        if shift_labels:
            lab = torch.full_like(labels, -100)
            lab[:, :-1] = labels[:, 1:]
        else:
            lab = labels
        if tp > 1:
            return self._vocab_parallel_loss(y, lab.reshape(-1))
        return O.lm_head_loss(y, self.head_weight(), lab.reshape(-1), softcap=cfg.final_softcap)

    # ---- vocab-parallel pieces (TP > 1) ------------------------------------------------------
    def _vocab_parallel_embed(self, ids, seq):
        cfg = self.cfg
        lo, hi = self.vocab_start, self.vocab_start + self.vocab_local
        mine = (ids >= lo) & (ids < hi)
        local = torch.where(mine, ids - lo, torch.zeros_like(ids))
        # with a sink the lookup gradient leaves as (rows of this vocabulary shard, values); tokens of other shards
        # map to row 0 with a zero gradient (their output is masked below)
        x = O.embedding(local, self.wte, None, seq, 0, cfg.embed_scale, self.sparse_sink)
        x = x * mine.unsqueeze(-1).to(x.dtype)
        x = O.reduce_from_tp(x, self.tp_group)
        if self.wpe is not None:
            x = x + self.wpe[cfg.pos_offset:cfg.pos_offset + seq].repeat(ids.numel() // seq, 1)
        return x

    def _logits(self, y):
        w = self.head_weight()
        logits = O.linear(y, w, None, "out_in")
        _, tp = _tp(self.tp_group)
        if tp > 1:
            parts = [torch.empty_like(logits) for _ in range(tp)]
            dist.all_gather(parts, logits.contiguous(), group=self.tp_group)
            logits = torch.cat(parts, dim=-1)
        return logits[..., : self.cfg.vocab_size]

    def _vocab_parallel_loss(self, y, labels):
        """Cross-entropy over vocabulary shards; the hidden-state gradient is the sum over the group of each shard's
        dlogits @ W_local (the input of this function is replicated, so that sum is its full gradient)."""
        return O.vocab_parallel_lm_head_loss(y, self.head_weight(), labels, self.tp_group, self.vocab_start,
                                             self.cfg.vocab_size, tp_ws=getattr(self, "tp_ws", None),
                                             softcap=self.cfg.final_softcap)

    def sync_replicated_grads(self):
        """Sum over the TP group the gradients of weights that are replicated but see only part of the work: the
        k / v projections when there are fewer KV heads than TP ranks (each rank back-propagates its own query
        heads through the same KV head)."""
        _, tp = _tp(self.tp_group)
        if tp == 1:
            return
        if getattr(self, "sequence_parallel", False):
            # parameters applied to this rank's token rows only: their gradients are partial sums over the group
            for p in self._sp_partial_params():
                if p.grad is not None:
                    dist.all_reduce(p.grad, group=self.tp_group)
        for b in self.blocks:
            if not b.kv_replicated or b.qkv_w.grad is None:
                continue
            lo = b.hq * self.cfg.head_dim
            gw = b.qkv_w.grad[:, lo:] if self.cfg.weight_layout == "in_out" else b.qkv_w.grad[lo:]
            buf = gw.contiguous()
            dist.all_reduce(buf, group=self.tp_group)
            gw.copy_(buf)
            if b.qkv_b is not None and b.qkv_b.grad is not None:
                dist.all_reduce(b.qkv_b.grad[lo:], group=self.tp_group)

    # ---- HuggingFace-format state dicts ---------------------------------------------------------
    def hf_state_dict(self) -> dict:
        from .hf_names import to_hf

        return to_hf(self)

    def load_hf_state_dict(self, sd: dict, strict: bool = True):
        from .hf_names import from_hf

        return from_hf(self, sd, strict)


def build_model(name_or_cfg, tp_group=None, device=None, dtype=torch.bfloat16, sparse_sink=None, **overrides) -> DecoderLM:
    from .config import get_config

    cfg = get_config(name_or_cfg, **overrides) if isinstance(name_or_cfg, str) else name_or_cfg
    return DecoderLM(cfg, tp_group, device, dtype, sparse_sink)
