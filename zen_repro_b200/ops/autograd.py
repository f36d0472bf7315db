"""Autograd wrappers that models are built from.  Each forwards to the raw ops (CUDA kernels on GPU,
PyTorch restatements on CPU), saves only what its hand-written backward needs, and never
materialises a transposed operand.
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import elementwise as E
from . import gemm as G
from . import attention as A

# the backward of an ungated activation also leaves the column sums of its result (the bias gradient of the layer before)
_FUSE_ACT_COLSUM = os.environ.get("ZEN_FUSE_ACT_COLSUM", "1") != "0"


def _claim(p, needed: bool) -> bool:
    """Called in forward.  True when this op will ADD its gradient for ``p`` straight into ``p.grad`` (a bucket
    view of the data-parallel reducer) and signal ``p.zen_ready``; the claim is counted so that the reducer knows
    how many such signals to expect before the parameter's bucket may be sent.  ``needed`` is the op's
    ``ctx.needs_input_grad`` entry for ``p``: grad mode itself is always off inside ``Function.forward``, so this is
    what tells a recorded forward from one under ``no_grad`` (the first pass of a checkpointed block)."""
    if p is None or not needed or not getattr(p, "zen_direct_grad", False) or p.grad is None:
        return False
    p.zen_expected = getattr(p, "zen_expected", 0) + 1
    return True


def _take_fresh(p) -> bool:
    """True once per step for a parameter whose bucket view has not been written yet in this step (the reducer marks
    it at ``zero_grad``).  The first direct writer then OVERWRITES instead of accumulating: the GEMM skips reading the
    old values, and the reducer does not have to zero the view between steps (it may still hold the last step's
    gradient)."""
    fresh = getattr(p, "zen_fresh", False)
    p.zen_fresh = False
    return fresh


def _declare_autograd_use(p, needed: bool) -> None:
    """Called in forward by an op whose gradient for ``p`` travels through autograd although other ops write
    theirs directly: the reducer then also waits for the accumulate-grad hook of ``p``."""
    if p is not None and needed and getattr(p, "zen_direct_grad", False):
        p.zen_autograd_use = True
        if getattr(p, "zen_fresh", False) and getattr(p, "zen_stale", False):
            p.grad.zero_()               # autograd accumulates: the view must not still hold the last step's gradient
            p.zen_stale = False


class LinearFn(torch.autograd.Function):
    """y = x @ W^T + b with W stored [out, in] ("out_in", nn.Linear) or [in, out] ("in_out", GPT-2 Conv1D).

    ``tp_mode`` selects a tensor-parallel variant whose all-reduce is fused into the GEMM epilogue through the
    workspace ``tp_ws``: "row" = the output is summed over the TP group (row-parallel layer; the bias is added once
    after the sum), "col" = the input gradient is summed over the TP group (column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, weight, bias, layout, tp_mode=None, tp_ws=None):
        ctx.layout = layout
        ctx.has_bias = bias is not None
        ctx.tp = (tp_mode, tp_ws)
        x2 = x.reshape(-1, x.shape[-1])
        n = weight.shape[0] if layout == "out_in" else weight.shape[1]
        if tp_mode == "row":
            y = tp_ws.gemm_ar_nt(x2, weight, bias) if layout == "out_in" else tp_ws.gemm_ar_nn(x2, weight, bias)
        elif layout == "out_in":
            y = G.gemm_nt(x2, weight, bias=bias)
        else:
            y = G.gemm_nn(x2, weight, bias=bias)
        ctx.save_for_backward(x2, weight)
        ctx.params = (weight, bias)
        ctx.direct = (_claim(weight, ctx.needs_input_grad[1]), _claim(bias, ctx.needs_input_grad[2]))
        ctx.xshape = x.shape
        return y if x.dim() == 2 else y.view(*x.shape[:-1], n)

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        tp_mode, tp_ws = ctx.tp
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            if tp_mode == "col":
                dx = tp_ws.gemm_ar_nn(dy2, weight) if ctx.layout == "out_in" else tp_ws.gemm_ar_nt(dy2, weight)
            else:
                dx = G.gemm_nn(dy2, weight) if ctx.layout == "out_in" else G.gemm_nt(dy2, weight)
            dx = dx.view(ctx.xshape)
        wp, bp = ctx.params
        if ctx.needs_input_grad[1]:
            a, b = (dy2, x2) if ctx.layout == "out_in" else (x2, dy2)
            if ctx.direct[0]:
                # written straight into the reducer's bucket view; may share one launch with the next few weight gradients
                G.defer_tn(a, b, wp.grad, accumulate=not _take_fresh(wp), done=lambda: wp.zen_ready(wp))
            else:
                dw = G.gemm_tn(a, b)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            # partial column sums that the producer of dy left beside it (ActFn.backward): dy is not read again
            part = getattr(dy, "_zen_colsum_part", None)
            if part is not None and (part.shape[1] != dy2.shape[1] or part.device != dy2.device):
                part = None
            if ctx.direct[1]:
                ready = lambda: bp.zen_ready(bp)     # after the (possibly queued) fold of the partial sums
                if part is not None:
                    E.colsum_from_parts(part, out=bp.grad, accumulate=not _take_fresh(bp), done=ready)
                else:
                    E.colsum(dy2, out=bp.grad, accumulate=not _take_fresh(bp), done=ready)
            elif part is not None:
                db = E.colsum_from_parts(part, torch.empty(dy2.shape[1], dtype=dy2.dtype, device=dy2.device), accumulate=False)
            else:
                db = E.colsum(dy2)
        return dx, dw, db, None, None, None


def linear(x, weight, bias=None, layout="out_in", tp_mode=None, tp_ws=None):
    return LinearFn.apply(x, weight, bias, layout, tp_mode, tp_ws)


class NormFn(torch.autograd.Function):
    """(y, h) = norm(x + residual): y feeds the next sub-layer, h is the updated residual stream."""

    @staticmethod
    def forward(ctx, x, residual, weight, bias, eps, layer, unit_offset):
        y, h, rstd, mean = E.norm_fwd(x, weight, bias, residual, eps=eps, layer=layer, unit_offset=unit_offset)
        ctx.save_for_backward(h, weight, rstd, mean if mean is not None else rstd)
        ctx.cfg = (layer, unit_offset, bias is not None, residual is not None)
        ctx.params = (weight, bias)
        # both or neither: the kernel produces the two column sums together
        both = ctx.needs_input_grad[2] and (bias is None or ctx.needs_input_grad[3])
        ctx.direct = both and _claim(weight, True) and (bias is None or _claim(bias, True))
        return y, h

    @staticmethod
    def backward(ctx, dy, dh_in):
        h, weight, rstd, mean = ctx.saved_tensors
        layer, unit_offset, has_bias, has_res = ctx.cfg
        wp, bp = ctx.params
        direct = ctx.direct
        acc = True
        if direct:
            fw, fb = _take_fresh(wp), (_take_fresh(bp) if bp is not None else None)
            acc = not fw
            if fb is not None and fb != fw:          # one of the pair was written before: zero the fresh one, then add
                (wp if fw else bp).grad.zero_()
                acc = True
        def ready():
            wp.zen_ready(wp)
            if bp is not None:
                bp.zen_ready(bp)

        dh, dw, db = E.norm_bwd(dy.contiguous(), h, weight, rstd, mean if layer else None, dh_in,
                                layer=layer, unit_offset=unit_offset, has_bias=has_bias,
                                dw_out=wp.grad if direct else None, db_out=bp.grad if (direct and bp is not None) else None,
                                accumulate=acc, done=ready if direct else None)
        if direct:
            dw = db = None
        return dh, (dh if has_res else None), dw, db, None, None, None


def fused_norm(x, residual, weight, bias=None, eps=1e-5, layer=False, unit_offset=False):
    return NormFn.apply(x, residual, weight, bias, eps, layer, unit_offset)


class ActFn(torch.autograd.Function):
    """Activation on a [.., inner] tensor, or gated activation on the two halves of a [.., 2 * inner] tensor."""

    @staticmethod
    def forward(ctx, x, kind):
        ctx.kind = kind
        gated = kind in ("swiglu", "geglu")
        x2 = x.reshape(-1, x.shape[-1])
        if gated:
            inner = x2.shape[1] // 2
            out = E.act_fwd(x2[:, :inner], x2[:, inner:], kind)
        else:
            inner = x2.shape[1]
            out = E.act_fwd(x2, None, kind)
        ctx.save_for_backward(x2)
        ctx.xshape = x.shape
        return out.view(*x.shape[:-1], inner)

    @staticmethod
    def backward(ctx, dout):
        (x2,) = ctx.saved_tensors
        kind = ctx.kind
        d2 = dout.reshape(-1, dout.shape[-1])
        part = None
        if kind in ("swiglu", "geglu"):
            dx = E.act_bwd_gated(x2, d2, kind)
        elif x2.is_cuda and x2.is_contiguous() and x2.shape[1] % 8 == 0 and _FUSE_ACT_COLSUM:
            dx, part = E.act_bwd_with_colsum(x2, d2, kind)
        else:
            dx, _ = E.act_bwd(x2, None, d2, kind)
        dx = dx.view(ctx.xshape)
        if part is not None:
            dx._zen_colsum_part = part       # read by the backward of the linear layer that receives dx as its dy
        return dx, None


def activation(x, kind):
    return ActFn.apply(x, kind)


class RopeFn(torch.autograd.Function):
    """Rotary embedding on the q and k parts of a fused [tokens, (Hq + 2 Hkv) * hd] projection, in place."""

    @staticmethod
    def forward(ctx, qkv, hq, hkv, hd, seq, theta):
        ctx.cfg = (hq, hkv, hd, seq, theta)
        t = qkv.shape[0]
        v3 = qkv.view(t, hq + 2 * hkv, hd)
        E.rope_(v3[:, :hq], seq, theta)
        E.rope_(v3[:, hq:hq + hkv], seq, theta)
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, d):
        hq, hkv, hd, seq, theta = ctx.cfg
        d = d.contiguous().clone() if not d.is_contiguous() else d.clone()
        v3 = d.view(d.shape[0], hq + 2 * hkv, hd)
        E.rope_(v3[:, :hq], seq, theta, inverse=True)
        E.rope_(v3[:, hq:hq + hkv], seq, theta, inverse=True)
        return d, None, None, None, None, None


def rope_qkv(qkv, hq, hkv, hd, seq, theta):
    return RopeFn.apply(qkv, hq, hkv, hd, seq, theta)


class EmbeddingFn(torch.autograd.Function):
    """Token (+ learned position) embedding.  With ``sparse_sink`` the lookup gradient is produced as
    (rows, count, values) and handed to the sink instead of being scattered into a dense [V, d] tensor."""

    @staticmethod
    def forward(ctx, ids, wte, wpe, seq, pos_offset, scale, sparse_sink, vocab_start):
        local = ids - vocab_start if vocab_start else ids
        if sparse_sink is None:
            _declare_autograd_use(wte, ctx.needs_input_grad[1])
        out = E.embedding_fwd(local, wte, wpe, seq=seq, pos_offset=pos_offset, scale=scale)
        ctx.save_for_backward(local)
        ctx.cfg = (wte.shape, wte.dtype, wpe.shape if wpe is not None else None, seq, pos_offset, scale, sparse_sink)
        return out

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        wshape, wdtype, pshape, seq, pos_offset, scale, sink = ctx.cfg
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dwpe = None
        if pshape is not None:
            bsz = dy2.shape[0] // seq
            dwpe = torch.zeros(pshape, dtype=dy.dtype, device=dy.device)
            dwpe[pos_offset:pos_offset + seq] = dy2.view(bsz, seq, -1).float().sum(0).to(dy.dtype)
        scratch = sink.scratch_for(ids.numel(), dy2) if sink is not None else None
        rows, count, vals = E.embedding_bwd_rows(ids, dy2, wshape[0], scale=scale, scratch=scratch)
        if sink is not None:
            sink.put(rows, count, vals)
            return None, None, dwpe, None, None, None, None, None
        dw = torch.zeros(wshape, dtype=wdtype, device=dy.device)
        E.rows_add_(dw, rows, count, vals)
        return None, dw, dwpe, None, None, None, None, None


def embedding(ids, wte, wpe=None, seq=1, pos_offset=0, scale=1.0, sparse_sink=None, vocab_start=0):
    return EmbeddingFn.apply(ids, wte, wpe, seq, pos_offset, scale, sparse_sink, vocab_start)


def _softcap_(logits: torch.Tensor, cap: float):
    """In place logits <- cap * tanh(logits / cap); returns tanh(logits / cap) for the gradient (None when off)."""
    if not cap or cap <= 0:
        return None
    th = torch.tanh(logits.float() / cap) if logits.dtype != torch.float32 else torch.tanh(logits / cap)
    logits.copy_(th * cap)
    return th


def _softcap_grad_(dlogits: torch.Tensor, th) -> None:
    """In place chain rule through the soft-capping: dlogits <- dlogits * (1 - tanh^2)."""
    if th is not None:
        dlogits.copy_(dlogits.float() * (1.0 - th * th))


class LMHeadLossFn(torch.autograd.Function):
    """mean cross-entropy(h @ W^T, labels).  Logits are computed, turned into dlogits in place by one
    kernel (already scaled by 1 / valid-token-count, read from the device), and immediately consumed
    by the two gradient GEMMs; only dh and dW survive the forward.  The incoming gradient of the loss
    is assumed to be 1 (``unit_grad``); otherwise the saved gradients are rescaled in backward."""

    @staticmethod
    def forward(ctx, h, weight, labels, ignore_index, chunk_tokens, unit_grad, softcap=0.0):
        h2 = h.reshape(-1, h.shape[-1])
        lab = labels.reshape(-1)
        T = h2.shape[0]
        inv = 1.0 / (lab != ignore_index).sum().clamp_(min=1).to(torch.float32).reshape(1)
        V = weight.shape[0]
        vpad = (V + 7) // 8 * 8
        dh = torch.empty_like(h2)
        direct = unit_grad and _claim(weight, ctx.needs_input_grad[1])
        if not direct:
            _declare_autograd_use(weight, ctx.needs_input_grad[1])
        nchunks = (T + chunk_tokens - 1) // chunk_tokens
        if direct:
            dw = weight.grad
        else:
            dw = torch.zeros(weight.shape, dtype=torch.float32 if (h2.is_cuda and nchunks > 1) else weight.dtype,
                             device=h2.device)
        loss_sum = torch.zeros((), dtype=torch.float32, device=h2.device)
        fresh = direct and _take_fresh(weight)
        for s in range(0, T, chunk_tokens):
            e = min(T, s + chunk_tokens)
            buf = torch.empty(e - s, vpad, dtype=h2.dtype, device=h2.device)
            logits = buf[:, :V]
            G.gemm_nt(h2[s:e], weight, out=logits, pad_ok=True)
            th = _softcap_(logits, softcap)
            loss, dl = E.cross_entropy(logits, lab[s:e], grad_scale=1.0, grad_scale_dev=inv, ignore_index=ignore_index)
            _softcap_grad_(dl, th)
            loss_sum += loss.sum()
            G.gemm_nn(dl, weight, out=dh[s:e])
            G.gemm_tn(dl, h2[s:e], out=dw, accumulate=not (fresh and s == 0))
        ctx.save_for_backward(dh, dw if not direct else dh)
        ctx.cfg = (h.shape, weight.dtype, direct, unit_grad)
        ctx.wp = weight
        return loss_sum * inv.squeeze(0)

    @staticmethod
    def backward(ctx, g):
        dh, dw = ctx.saved_tensors
        hshape, wdtype, direct, unit = ctx.cfg
        if direct:
            ctx.wp.zen_ready(ctx.wp)
            return dh.view(hshape), None, None, None, None, None, None
        if unit:
            return dh.view(hshape), dw.to(wdtype), None, None, None, None, None
        return (dh.float() * g).to(dh.dtype).view(hshape), (dw.float() * g).to(wdtype), None, None, None, None, None


def lm_head_loss(h, weight, labels, ignore_index=-100, chunk_tokens=8192, unit_grad=True, softcap: float = 0.0):
    """``softcap`` > 0: logits -> cap * tanh(logits / cap) before the loss (Gemma-2's final-logit soft-capping)."""
    return LMHeadLossFn.apply(h, weight, labels, ignore_index, chunk_tokens, unit_grad, softcap)


class VocabParallelLMHeadLossFn(torch.autograd.Function):
    """LM head + cross-entropy with the vocabulary sharded over the tensor-parallel group.  Per chunk of tokens: local
    logits GEMM, local max / sum-exp / target logit (one kernel), three [tokens]-sized all-reduces, dlogits in place
    (one kernel), then dW_local = dlogits^T h and the partial dh = dlogits W_local, which is summed over the group
    (fused into the GEMM epilogue when a workspace is given).  Unit incoming gradient assumed, as in LMHeadLossFn."""

    @staticmethod
    def forward(ctx, h, weight, labels, group, vocab_start, vocab_size, ignore_index, chunk_tokens, tp_ws, softcap=0.0):
        h2 = h.reshape(-1, h.shape[-1])
        lab = labels.reshape(-1)
        T = h2.shape[0]
        Vl = weight.shape[0]
        valid_cols = max(0, min(Vl, vocab_size - vocab_start))
        inv = 1.0 / (lab != ignore_index).sum().clamp_(min=1).to(torch.float32).reshape(1)
        vpad = (Vl + 7) // 8 * 8
        dh = torch.empty_like(h2)
        direct = _claim(weight, ctx.needs_input_grad[1])
        if not direct:
            _declare_autograd_use(weight, ctx.needs_input_grad[1])
        dw = weight.grad if direct else torch.zeros(weight.shape, dtype=weight.dtype, device=h2.device)
        loss_sum = torch.zeros((), dtype=torch.float32, device=h2.device)
        fresh = direct and _take_fresh(weight)
        for s in range(0, T, chunk_tokens):
            e = min(T, s + chunk_tokens)
            buf = torch.empty(e - s, vpad, dtype=h2.dtype, device=h2.device)
            logits = buf[:, :Vl]
            G.gemm_nt(h2[s:e], weight, out=logits, pad_ok=True)
            th = _softcap_(logits, softcap)
            m, se, tgt = E.xent_partial(logits, lab[s:e], valid_cols, vocab_start, ignore_index)
            gm = m.clone()
            dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=group)
            se = se * torch.exp(m - gm)
            packed = torch.stack([se, tgt])
            dist.all_reduce(packed, group=group)
            lse = gm + packed[0].log()
            valid = lab[s:e] != ignore_index
            loss_sum += ((lse - packed[1]) * valid).sum()
            E.xent_apply_(logits, lab[s:e], lse, valid_cols, vocab_start, grad_scale_dev=inv, ignore_index=ignore_index)
            _softcap_grad_(logits, th)
            if tp_ws is not None and tp_ws.fits(e - s, h2.shape[1]):
                tp_ws.gemm_ar_nn(logits, weight, out=dh[s:e])
            else:
                part = G.gemm_nn(logits, weight)
                dist.all_reduce(part, group=group)
                dh[s:e] = part
            G.gemm_tn(logits, h2[s:e], out=dw, accumulate=not (fresh and s == 0))
        ctx.save_for_backward(dh, dw if not direct else dh)
        ctx.cfg = (h.shape, direct)
        ctx.wp = weight
        return loss_sum * inv.squeeze(0)

    @staticmethod
    def backward(ctx, g):
        dh, dw = ctx.saved_tensors
        hshape, direct = ctx.cfg
        if direct:
            ctx.wp.zen_ready(ctx.wp)
            return (dh.view(hshape),) + (None,) * 9
        return (dh.view(hshape), dw) + (None,) * 8


def vocab_parallel_lm_head_loss(h, weight, labels, group, vocab_start, vocab_size, ignore_index=-100, chunk_tokens=8192,
                                tp_ws=None, softcap: float = 0.0):
    return VocabParallelLMHeadLossFn.apply(h, weight, labels, group, vocab_start, vocab_size, ignore_index, chunk_tokens,
                                           tp_ws, softcap)


class AttentionFn(torch.autograd.Function):
    """Causal self-attention over a fused qkv projection [B*S, (Hq + 2 Hkv) * hd] -> [B*S, Hq * hd]."""

    @staticmethod
    def forward(ctx, qkv, bsz, seq, hq, hkv, hd, scale, softcap):
        out, saved = A.attention_fwd(qkv, bsz, seq, hq, hkv, hd, scale, softcap)
        ctx.save_for_backward(qkv, out, *saved)
        ctx.cfg = (bsz, seq, hq, hkv, hd, scale, softcap)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, *saved = ctx.saved_tensors
        dqkv = A.attention_bwd(dout.contiguous(), qkv, out, saved, *ctx.cfg)
        return (dqkv,) + (None,) * 7


class PaddedAttentionFn(torch.autograd.Function):
    """The same attention for a head size or sequence length that the kernels do not take directly: zero-pad to the
    next covered shape, run the kernels there, cut the result back."""

    @staticmethod
    def forward(ctx, qkv, bsz, seq, hq, hkv, hd, scale, softcap, seq_p, hd_p):
        qp = A.pad_qkv(qkv, bsz, seq, hq + 2 * hkv, hd, seq_p, hd_p)
        out_p, lse2 = A.attention_fwd_kernel(qp, bsz, seq_p, hq, hkv, hd_p, scale, softcap)
        ctx.save_for_backward(qp, out_p, lse2)
        ctx.cfg = (bsz, seq, hq, hkv, hd, scale, softcap, seq_p, hd_p)
        return A.unpad(out_p, bsz, seq, hq, hd, seq_p, hd_p)

    @staticmethod
    def backward(ctx, dout):
        qp, out_p, lse2 = ctx.saved_tensors
        bsz, seq, hq, hkv, hd, scale, softcap, seq_p, hd_p = ctx.cfg
        dp = A.pad_qkv(dout.contiguous(), bsz, seq, hq, hd, seq_p, hd_p)
        dqkv_p = A.attention_bwd_kernel(dp, qp, out_p, lse2, bsz, seq_p, hq, hkv, hd_p, scale, softcap)
        return (A.unpad(dqkv_p, bsz, seq, hq + 2 * hkv, hd, seq_p, hd_p),) + (None,) * 9


def attention(qkv, bsz, seq, hq, hkv, hd, scale=None, softcap: float = 0.0):
    """``softcap`` > 0: scores are soft-capped, cap * tanh(s * scale / cap), before the softmax (Gemma-2)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if qkv.is_cuda and not A.have_kernel(seq, hq, hkv, hd, qkv.dtype, softcap):
        pad = A.padded_shape(seq, hq, hkv, hd, qkv.dtype, softcap)
        if pad is not None:
            return PaddedAttentionFn.apply(qkv, bsz, seq, hq, hkv, hd, scale, softcap, *pad)
        if softcap > 0:
            return A.reference_attention(qkv, bsz, seq, hq, hkv, hd, scale, softcap)
        # library fallback under plain autograd (keeps the forward's softmax statistics, no recompute)
        q, k, v = A._split(qkv, bsz, seq, hq, hkv, hd)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale, enable_gqa=(hq != hkv))
        return o.transpose(1, 2).reshape(bsz * seq, hq * hd)
    return AttentionFn.apply(qkv, bsz, seq, hq, hkv, hd, scale, softcap)


# ------------------------------------------------------------------------------------------ tensor parallel
class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel linear)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel linear)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


# ---- sequence parallelism: the residual stream is sharded over the tokens of the TP group ------------------------
def _gather_rows(x, group):
    """[T / P, C] on every rank -> [T, C] (rank-major row blocks)."""
    P = dist.get_world_size(group)
    x = x.contiguous()
    out = torch.empty(P * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def _reduce_scatter_rows(x, group):
    """[T, C] partial sums on every rank -> this rank's [T / P, C] rows of the sum."""
    P, r = dist.get_world_size(group), dist.get_rank(group)
    x = x.contiguous()
    n = x.shape[0] // P
    if not x.is_cuda:                      # gloo has no reduce-scatter
        dist.all_reduce(x, group=group)
        return x[r * n:(r + 1) * n].clone()
    out = torch.empty(n, *x.shape[1:], dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


class _ScatterToSP(torch.autograd.Function):
    """Keep this rank's block of token rows (forward); all-gather the row gradients (backward)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        P, r = dist.get_world_size(group), dist.get_rank(group)
        n = x.shape[0] // P
        return x[r * n:(r + 1) * n].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _gather_rows(g, ctx.group), None


class _GatherFromSP(torch.autograd.Function):
    """All-gather the token rows (forward); keep this rank's block of the gradient (backward).  The consumer is a
    vocabulary-parallel head whose input gradient is already summed over the group, hence identical on every rank."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _gather_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        P, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        n = g.shape[0] // P
        return g[r * n:(r + 1) * n].contiguous(), None


def scatter_to_sp(x, group):
    return _ScatterToSP.apply(x, group)


def gather_from_sp(x, group):
    return _GatherFromSP.apply(x, group)


class SPLinearFn(torch.autograd.Function):
    """Linear layer of a sequence-parallel block.

    mode "ag" (column-parallel weight): the input is this rank's token rows; y = all_gather(x) @ W^T has all tokens
    and this rank's output columns.  mode "rs" (row-parallel weight): the input has all tokens and this rank's
    slice of the contraction; y = reduce_scatter(x @ W^T) is this rank's token rows of the summed product (+ bias,
    once).  With a ``FusedTPWorkspace`` on CUDA the forward of both and the input gradient of "ag" run as one kernel
    (``ag_gemm_*`` / ``gemm_rs_*``: GEMM and collective over peer memory); the operand that a weight gradient needs
    in full (x for "ag", dy for "rs") is all-gathered in backward, as Megatron-style sequence parallelism does."""

    @staticmethod
    def forward(ctx, x, weight, bias, layout, mode, group, ws):
        x2 = x.reshape(-1, x.shape[-1])
        P = dist.get_world_size(group)
        out_in = layout == "out_in"
        n = weight.shape[0] if out_in else weight.shape[1]
        fused = ws is not None and x2.is_cuda and x2.dtype == torch.bfloat16
        if mode == "ag":
            if fused and ws.fits_ag(x2.shape[0], x2.shape[1], n):
                y = ws.ag_gemm_nt(x2, weight, bias) if out_in else ws.ag_gemm_nn(x2, weight, bias)
            else:
                xf = _gather_rows(x2, group)
                y = G.gemm_nt(xf, weight, bias=bias) if out_in else G.gemm_nn(xf, weight, bias=bias)
        else:
            if fused and ws.fits_rs(x2.shape[0], n):
                y = ws.gemm_rs_nt(x2, weight, bias) if out_in else ws.gemm_rs_nn(x2, weight, bias)
            else:
                y = G.gemm_nt(x2, weight) if out_in else G.gemm_nn(x2, weight)
                y = _reduce_scatter_rows(y, group)
                if bias is not None:
                    y = y + bias
        ctx.save_for_backward(x2, weight)
        ctx.cfg = (layout, mode, group, ws, bias is not None)
        ctx.params = (weight, bias)
        ctx.direct = (_claim(weight, ctx.needs_input_grad[1]), _claim(bias, ctx.needs_input_grad[2]))
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        layout, mode, group, ws, has_bias = ctx.cfg
        out_in = layout == "out_in"
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        fused = ws is not None and dy2.is_cuda and dy2.dtype == torch.bfloat16
        dx = dw = db = None
        wp, bp = ctx.params
        if mode == "ag":
            # dx: every rank holds a partial [T, K] (its output columns); this rank needs its token rows of the sum
            if ctx.needs_input_grad[0]:
                if fused and ws.fits_rs(dy2.shape[0], x2.shape[1]):
                    dx = ws.gemm_rs_nn(dy2, weight) if out_in else ws.gemm_rs_nt(dy2, weight)
                else:
                    part = G.gemm_nn(dy2, weight) if out_in else G.gemm_nt(dy2, weight)
                    dx = _reduce_scatter_rows(part, group)
            xf = _gather_rows(x2, group) if ctx.needs_input_grad[1] else None
            dyf, db_src = dy2, dy2
        else:
            dyf = _gather_rows(dy2, group)
            if ctx.needs_input_grad[0]:
                dx = G.gemm_nn(dyf, weight) if out_in else G.gemm_nt(dyf, weight)
            xf, db_src = x2, dy2                 # the bias gradient of this rank covers its token rows only
        if ctx.needs_input_grad[1]:
            a, b = (dyf, xf) if out_in else (xf, dyf)
            if ctx.direct[0]:
                G.gemm_tn(a, b, out=wp.grad, accumulate=not _take_fresh(wp))
                wp.zen_ready(wp)
            else:
                dw = G.gemm_tn(a, b)
        if has_bias and ctx.needs_input_grad[2]:
            if ctx.direct[1]:
                E.colsum(db_src, out=bp.grad, accumulate=not _take_fresh(bp))
                bp.zen_ready(bp)
            else:
                db = E.colsum(db_src)
        return dx, dw, db, None, None, None, None


def sp_linear(x, weight, bias, layout, mode, group, ws=None):
    return SPLinearFn.apply(x, weight, bias, layout, mode, group, ws)


def copy_to_tp(x, group):
    return x if group is None or dist.get_world_size(group) == 1 else _CopyToTP.apply(x, group)


def reduce_from_tp(x, group):
    return x if group is None or dist.get_world_size(group) == 1 else _ReduceFromTP.apply(x, group)
