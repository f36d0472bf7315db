"""Causal self-attention (MHA / GQA / MQA) over a fused qkv buffer.

The raw entry points take the fused projection ``qkv[B*S, (Hq + 2*Hkv)*hd]`` and return
``out[B*S, Hq*hd]``.  On CUDA, bf16 forward and backward run on the tcgen05 flash kernels of
``csrc/attention_tcgen05.cu`` (head_dim 64 / 128 / 256, sequence a multiple of 128); other head sizes up
to 256 and other sequence lengths are zero-padded to the next covered shape (``padded_shape``): padded
head columns add nothing to any dot product, and padded positions sit at the end, where the causal mask
hides them from every real query and their zero output gradient adds nothing to dK / dV.  On CPU a plain
softmax(QK^T)V restatement is used, which is also the oracle for tests.  The library attention is reached
only for other dtypes or when forced with ``ZEN_ATTN=lib``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


import ctypes
import os

from .. import _native

_MODE = os.environ.get("ZEN_ATTN", "auto")        # auto | own | lib


def kernel_covers(seq, hq, hkv, hd, dtype, backward: bool = False) -> bool:
    """Shapes the tcgen05 attention kernels handle."""
    if dtype != torch.bfloat16 or seq % 128 or hq % hkv:
        return False
    return hd in (64, 128, 256)


def have_kernel(seq, hq, hkv, hd, dtype, softcap: float = 0.0) -> bool:
    """True when forward AND backward run on the hand-written kernels for this shape (soft-capped scores: the
    head_dim 256 kernels only; other head sizes are padded to 256)."""
    if _MODE == "lib":
        return False
    if softcap > 0 and hd != 256:
        return False
    return kernel_covers(seq, hq, hkv, hd, dtype, backward=True) and HAVE_BWD


HAVE_BWD = True


def padded_shape(seq, hq, hkv, hd, dtype, softcap: float = 0.0):
    """(seq', hd') of the covered shape that (seq, hd) is zero-padded to, or None when padding cannot help."""
    if _MODE == "lib" or dtype != torch.bfloat16 or hq % hkv or hd > 256 or not HAVE_BWD:
        return None
    return (seq + 127) // 128 * 128, (256 if softcap > 0 else next(h for h in (64, 128, 256) if h >= hd))


def pad_qkv(qkv, bsz, seq, nheads, hd, seq_p, hd_p):
    """[B*S, nheads*hd] -> zero-padded [B*S', nheads*hd'] (contiguous)."""
    out = qkv.new_zeros(bsz, seq_p, nheads, hd_p)
    out[:, :seq, :, :hd] = qkv.view(bsz, seq, nheads, hd)
    return out.view(bsz * seq_p, nheads * hd_p)


def unpad(t, bsz, seq, nheads, hd, seq_p, hd_p):
    return t.view(bsz, seq_p, nheads, hd_p)[:, :seq, :, :hd].reshape(bsz * seq, nheads * hd)


def attention_fwd_kernel(qkv, bsz, seq, hq, hkv, hd, scale, softcap: float = 0.0):
    """tcgen05 forward: returns (out[B*S, Hq*hd], lse2[B, Hq, S]) with lse2 in base 2 of the scaled scores.
    ``softcap`` > 0 soft-caps the scaled scores, cap * tanh(s / cap), before the softmax (Gemma-2)."""
    assert qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1
    out = torch.empty(bsz * seq, hq * hd, dtype=qkv.dtype, device=qkv.device)
    lse2 = torch.empty(bsz, hq, seq, dtype=torch.float32, device=qkv.device)
    rc = _native.lib().zen_attn_fwd(_native.ptr(qkv), _native.ptr(out), _native.ptr(lse2), bsz, seq, hq, hkv, hd,
                                    qkv.stride(0), out.stride(0), ctypes.c_float(scale), ctypes.c_float(softcap),
                                    _native.stream_ptr())
    _native.check(rc, "zen_attn_fwd")
    return out, lse2


_BWD64 = os.environ.get("ZEN_ATTN_BWD64", "")      # "", or 0 / 1 / 2: which head_dim 64 backward kernels run (measurements)
_bwd64_applied = False


def attention_bwd_kernel(dout, qkv, out, lse2, bsz, seq, hq, hkv, hd, scale, softcap: float = 0.0):
    """tcgen05 backward: gradient of the fused qkv buffer (dQ kernel + dK/dV kernel, no atomics)."""
    global _bwd64_applied
    if _BWD64 and not _bwd64_applied:
        _native.lib().zen_attn_bwd64_variant(int(_BWD64))
        _bwd64_applied = True
    dout = dout if (dout.is_contiguous() and dout.data_ptr() % 16 == 0) else dout.contiguous()
    dqkv = torch.empty_like(qkv)
    dbuf = torch.empty(bsz, hq, seq, dtype=torch.float32, device=qkv.device)
    hsplit, part = 1, None
    rep = hq // hkv
    if hd == 256 and rep > 1:
        # few KV heads (MQA / GQA): spread the query heads of a group over several CTAs until the GPU is covered
        base = hkv * bsz * (seq // 128)
        hsplit = next((d for d in range(1, rep + 1) if rep % d == 0 and base * d >= 2 * 148), rep)
        if hsplit > 1:
            part = torch.empty(2 * hsplit * bsz * seq * hkv * 256, dtype=torch.float32, device=qkv.device)
    rc = _native.lib().zen_attn_bwd(_native.ptr(qkv), _native.ptr(out), _native.ptr(dout), _native.ptr(lse2), _native.ptr(dbuf),
                                    _native.ptr(dqkv), bsz, seq, hq, hkv, hd, qkv.stride(0), out.stride(0),
                                    ctypes.c_float(scale), ctypes.c_float(softcap), _native.ptr(part), hsplit,
                                    _native.stream_ptr())
    _native.check(rc, "zen_attn_bwd")
    return dqkv


def attention_error() -> int:
    return int(_native.lib().zen_attn_error())


def _split(qkv, bsz, seq, hq, hkv, hd):
    t = qkv.view(bsz, seq, hq + 2 * hkv, hd)
    q = t[:, :, :hq].transpose(1, 2)
    k = t[:, :, hq:hq + hkv].transpose(1, 2)
    v = t[:, :, hq + hkv:].transpose(1, 2)
    return q, k, v


def reference_attention(qkv, bsz, seq, hq, hkv, hd, scale, softcap: float = 0.0):
    q, k, v = _split(qkv.float(), bsz, seq, hq, hkv, hd)
    rep = hq // hkv
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    s = (q @ k.transpose(-1, -2)) * scale
    if softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    mask = torch.ones(seq, seq, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    o = torch.softmax(s, -1) @ v
    return o.transpose(1, 2).reshape(bsz * seq, hq * hd).to(qkv.dtype)


def attention_fwd(qkv, bsz, seq, hq, hkv, hd, scale, softcap: float = 0.0):
    if not qkv.is_cuda:
        return reference_attention(qkv, bsz, seq, hq, hkv, hd, scale, softcap), ()
    if have_kernel(seq, hq, hkv, hd, qkv.dtype) and qkv.is_contiguous():
        out, lse2 = attention_fwd_kernel(qkv, bsz, seq, hq, hkv, hd, scale, softcap)
        return out, (lse2,)
    if softcap > 0:
        return reference_attention(qkv, bsz, seq, hq, hkv, hd, scale, softcap), ()
    q, k, v = _split(qkv, bsz, seq, hq, hkv, hd)
    o = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale, enable_gqa=(hq != hkv))
    return o.transpose(1, 2).reshape(bsz * seq, hq * hd), ()


def attention_bwd(dout, qkv, out, saved, bsz, seq, hq, hkv, hd, scale, softcap: float = 0.0):
    """Gradient w.r.t. the fused qkv buffer: the tcgen05 kernels when the forward saved its statistics, else a
    recomputation under autograd."""
    if len(saved) == 1 and qkv.is_cuda:
        return attention_bwd_kernel(dout, qkv, out, saved[0], bsz, seq, hq, hkv, hd, scale, softcap)
    with torch.enable_grad():
        x = qkv.detach().requires_grad_(True)
        if not qkv.is_cuda or softcap > 0:
            o = reference_attention(x, bsz, seq, hq, hkv, hd, scale, softcap)
        else:
            q, k, v = _split(x, bsz, seq, hq, hkv, hd)
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale, enable_gqa=(hq != hkv))
            o = o.transpose(1, 2).reshape(bsz * seq, hq * hd)
        (g,) = torch.autograd.grad(o, x, dout)
    return g
