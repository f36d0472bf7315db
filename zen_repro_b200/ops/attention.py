"""Causal self-attention (MHA / GQA / MQA) over a fused qkv buffer.

The raw entry points take the fused projection ``qkv[B*S, (Hq + 2*Hkv)*hd]`` and return
``out[B*S, Hq*hd]``.  On CUDA the forward and backward run through
``torch.nn.functional.scaled_dot_product_attention`` (library flash kernels) until the tcgen05
attention kernels in ``csrc/`` cover the shape; on CPU a plain softmax(QK^T)V restatement is used,
which is also the oracle for tests.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def have_kernel(seq, hq, hkv, hd, dtype) -> bool:
    """True when the hand-written attention kernels cover this shape."""
    return False


def _split(qkv, bsz, seq, hq, hkv, hd):
    t = qkv.view(bsz, seq, hq + 2 * hkv, hd)
    q = t[:, :, :hq].transpose(1, 2)
    k = t[:, :, hq:hq + hkv].transpose(1, 2)
    v = t[:, :, hq + hkv:].transpose(1, 2)
    return q, k, v


def reference_attention(qkv, bsz, seq, hq, hkv, hd, scale):
    q, k, v = _split(qkv.float(), bsz, seq, hq, hkv, hd)
    rep = hq // hkv
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    s = (q @ k.transpose(-1, -2)) * scale
    mask = torch.ones(seq, seq, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    o = torch.softmax(s, -1) @ v
    return o.transpose(1, 2).reshape(bsz * seq, hq * hd).to(qkv.dtype)


def attention_fwd(qkv, bsz, seq, hq, hkv, hd, scale):
    if not qkv.is_cuda:
        return reference_attention(qkv, bsz, seq, hq, hkv, hd, scale), ()
    q, k, v = _split(qkv, bsz, seq, hq, hkv, hd)
    o = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale, enable_gqa=(hq != hkv))
    return o.transpose(1, 2).reshape(bsz * seq, hq * hd), ()


def attention_bwd(dout, qkv, out, saved, bsz, seq, hq, hkv, hd, scale):
    """Gradient w.r.t. the fused qkv buffer (recomputes the forward under autograd)."""
    with torch.enable_grad():
        x = qkv.detach().requires_grad_(True)
        if not qkv.is_cuda:
            o = reference_attention(x, bsz, seq, hq, hkv, hd, scale)
        else:
            q, k, v = _split(x, bsz, seq, hq, hkv, hd)
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale, enable_gqa=(hq != hkv))
            o = o.transpose(1, 2).reshape(bsz * seq, hq * hd)
        (g,) = torch.autograd.grad(o, x, dout)
    return g
