"""Raw (non-autograd) functional forms of the memory-bound model ops.

Every function dispatches on the device of its inputs: CUDA tensors run the
hand-written kernels in ``csrc/elementwise_kernels.cu``; CPU tensors run the
PyTorch restatement in the same function, which is also the oracle of the GPU
tests.  The autograd wrappers that models use live in ``ops/autograd.py``.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from .. import _native

ACT_GELU_TANH, ACT_RELU, ACT_SILU_GATE, ACT_GELU_GATE = 0, 1, 2, 3
_ACT = {"gelu_tanh": 0, "relu": 1, "swiglu": 2, "geglu": 3}

_scratch: dict = {}


def _scratch_buf(key, numel: int, dtype, device) -> torch.Tensor:
    """Per-(purpose, device, stream) scratch that grows but is never freed."""
    k = (key, device, dtype, torch.cuda.current_stream().cuda_stream)
    buf = _scratch.get(k)
    if buf is None or buf.numel() < numel:
        buf = torch.empty(max(numel, 1), dtype=dtype, device=device)
        _scratch[k] = buf
    return buf


def _code(t: torch.Tensor) -> int:
    return _native.DTYPE_CODE[t.dtype]


def _c(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


# ----------------------------------------------------------------------------- norms
def norm_fwd(x, weight, bias=None, residual=None, *, eps=1e-5, layer=False, unit_offset=False, want_h=True):
    """h = x (+ residual); y = norm(h).  Returns (y, h, rstd, mean) -- h is x itself without a residual."""
    cols = x.shape[-1]
    x2 = _c(x).view(-1, cols)
    rows = x2.shape[0]
    if not x.is_cuda:
        h = x2.float() + (residual.reshape(-1, cols).float() if residual is not None else 0)
        h = h.to(x.dtype)                     # the residual stream is stored in the activation dtype
        hf = h.float()
        if layer:
            mean = hf.mean(-1)
            var = hf.var(-1, unbiased=False)
            rstd = torch.rsqrt(var + eps)
            y = (hf - mean[:, None]) * rstd[:, None] * weight.float() + (bias.float() if bias is not None else 0)
        else:
            mean = None
            rstd = torch.rsqrt(hf.pow(2).mean(-1) + eps)
            w = weight.float() + 1.0 if unit_offset else weight.float()
            y = hf * rstd[:, None] * w
        return y.to(x.dtype).view(x.shape), h.view(x.shape), rstd, mean
    y = torch.empty_like(x2)
    res2 = _c(residual).view(-1, cols) if residual is not None else None
    h = torch.empty_like(x2) if residual is not None else x2
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device) if layer else None
    rc = _native.lib().zen_norm_fwd(_native.ptr(x2), _native.ptr(res2), _native.ptr(weight), _native.ptr(bias),
                                    _native.ptr(y), _native.ptr(h if residual is not None else None),
                                    _native.ptr(rstd), _native.ptr(mean), rows, cols, ctypes.c_float(eps),
                                    int(layer), int(unit_offset), _code(x2), _native.stream_ptr())
    _native.check(rc, "zen_norm_fwd")
    return y.view(x.shape), h.view(x.shape), rstd, mean


def norm_bwd(dy, h, weight, rstd, mean=None, dres=None, *, layer=False, unit_offset=False, has_bias=False,
             dw_out=None, db_out=None, accumulate=True, done=None):
    """Returns (dh, dweight, dbias): dh includes ``dres`` (gradient on the residual stream) when given.
    With ``dw_out`` / ``db_out`` the parameter gradients are added into those tensors instead (``accumulate``) or
    overwrite them."""
    cols = h.shape[-1]
    dy2, h2 = _c(dy).view(-1, cols), _c(h).view(-1, cols)
    rows = h2.shape[0]
    if not h.is_cuda:
        hf, g = h2.float(), dy2.float()
        if layer:
            xh = (hf - mean[:, None]) * rstd[:, None]
            gw = g * weight.float()
            dh = rstd[:, None] * (gw - gw.mean(-1, keepdim=True) - xh * (gw * xh).mean(-1, keepdim=True))
        else:
            xh = hf * rstd[:, None]
            w = weight.float() + 1.0 if unit_offset else weight.float()
            gw = g * w
            dh = rstd[:, None] * (gw - xh * (gw * xh).mean(-1, keepdim=True))
        dw = (g * xh).sum(0).to(weight.dtype)
        db = g.sum(0).to(weight.dtype) if (layer and has_bias) else None
        if dres is not None:
            dh = dh + dres.reshape(-1, cols).float()
        if dw_out is not None:
            dw_out.add_(dw) if accumulate else dw_out.copy_(dw)
            dw = dw_out
        if db_out is not None and db is not None:
            db_out.add_(db) if accumulate else db_out.copy_(db)
            db = db_out
        if done is not None:
            done()
        return dh.to(h.dtype).view(h.shape), dw, db
    lib = _native.lib()
    dh = torch.empty_like(h2)
    acc = dw_out is not None and accumulate
    dw = dw_out if dw_out is not None else torch.empty_like(weight)
    db = (db_out if db_out is not None else torch.empty_like(weight)) if (layer and has_bias) else None
    dres2 = _c(dres).view(-1, cols) if dres is not None else None
    if dw_out is not None and (db is None or db_out is not None) and _may_defer(done):
        # partial sums now, the fold into dw / db with the layer's other reductions
        used = lib.zen_norm_bwd_parts_used(rows, cols)
        part_dw = torch.empty(used, cols, dtype=torch.float32, device=h.device)
        part_db = torch.empty(used, cols, dtype=torch.float32, device=h.device) if layer else None
        rc = lib.zen_norm_bwd_ex(_native.ptr(dy2), _native.ptr(h2), _native.ptr(weight), _native.ptr(rstd), _native.ptr(mean),
                                 _native.ptr(dres2), _native.ptr(dh), _native.ptr(part_dw), _native.ptr(part_db),
                                 _native.ptr(dw), _native.ptr(db), rows, cols, int(layer), int(unit_offset), int(acc),
                                 _code(h2), 1, _native.stream_ptr())
        _native.check(rc, "zen_norm_bwd_ex")
        _queue_reduce(part_dw, used, dw, acc, done, part_db if db is not None else None, db)
        return dh.view(h.shape), dw, db
    parts = lib.zen_norm_bwd_parts(rows)
    part_dw = _scratch_buf("norm_dw", parts * cols, torch.float32, h.device)
    part_db = _scratch_buf("norm_db", parts * cols, torch.float32, h.device) if layer else None
    rc = lib.zen_norm_bwd(_native.ptr(dy2), _native.ptr(h2), _native.ptr(weight), _native.ptr(rstd), _native.ptr(mean),
                          _native.ptr(dres2), _native.ptr(dh), _native.ptr(part_dw), _native.ptr(part_db),
                          _native.ptr(dw), _native.ptr(db), rows, cols, int(layer), int(unit_offset), int(acc), _code(h2),
                          _native.stream_ptr())
    _native.check(rc, "zen_norm_bwd")
    if done is not None:
        done()
    return dh.view(h.shape), dw, db


# ---------------------------------------------------------------------------------------------------------------
# Deferred column reductions.  A bias or norm-parameter gradient is a two-step sum: per-row-group partials [parts, cols]
# (written by the kernel that has the data), then a tiny kernel that folds the parts into the gradient.  Inside a
# backward pass the second step may be queued (``done`` given): the queue goes out as ONE launch of up to eight
# reductions together with the grouped weight gradients (ops/gemm.py:flush_deferred), instead of six launches of a
# few microseconds per layer.
class _ReduceJob(ctypes.Structure):
    _fields_ = [("part", ctypes.c_void_p), ("out", ctypes.c_void_p), ("part2", ctypes.c_void_p), ("out2", ctypes.c_void_p),
                ("nparts", ctypes.c_int32), ("cols", ctypes.c_int32), ("accumulate", ctypes.c_int32), ("pad", ctypes.c_int32)]


_reduce_jobs: list = []


def _may_defer(done) -> bool:
    from . import gemm as _G

    return done is not None and _G.GROUP_SIZE > 1 and _G.arm_flush_at_end_of_backward()


def _queue_reduce(part, nparts, out, accumulate, done, part2=None, out2=None) -> None:
    ptrs = {out.data_ptr()} | ({out2.data_ptr()} if out2 is not None else set())
    clash = any(j[2].data_ptr() in ptrs or (j[6] is not None and j[6].data_ptr() in ptrs) for j in _reduce_jobs)
    if _reduce_jobs and (clash or _reduce_jobs[0][2].dtype != out.dtype or _reduce_jobs[0][2].device != out.device):
        flush_colreduce()                          # one launch never holds two reductions into one gradient
    _reduce_jobs.append((part, nparts, out, bool(accumulate), done, part2, out2))
    if len(_reduce_jobs) >= _native.lib().zen_colreduce_max_jobs():
        flush_colreduce()


def flush_colreduce() -> None:
    """Launch the queued column reductions (one launch) and run their callbacks."""
    if not _reduce_jobs:
        return
    jobs = list(_reduce_jobs)
    _reduce_jobs.clear()
    arr = (_ReduceJob * len(jobs))()
    for i, (part, nparts, out, acc, _done, part2, out2) in enumerate(jobs):
        arr[i] = _ReduceJob(part.data_ptr(), out.data_ptr(), part2.data_ptr() if part2 is not None else None,
                            out2.data_ptr() if out2 is not None else None, nparts, out.numel(), int(acc), 0)
    _native.check(_native.lib().zen_colreduce_multi(arr, len(jobs), _code(jobs[0][2]), _native.stream_ptr()),
                  "zen_colreduce_multi")
    for job in jobs:
        if job[4] is not None:
            job[4]()


def colsum(a: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = True, done=None) -> torch.Tensor:
    """Column sums of a [rows, cols] matrix (bias gradients); added into ``out`` when given (``accumulate``) or written
    over it.  ``done``: called once ``out`` has been (or, inside a backward pass, has been queued to be and then was)
    written; see the deferred reductions above."""
    cols = a.shape[-1]
    a2 = _c(a).view(-1, cols)
    if not a.is_cuda:
        r = a2.float().sum(0).to(a.dtype)
        r = r if out is None else (out.add_(r) if accumulate else out.copy_(r))
        if done is not None:
            done()
        return r
    lib = _native.lib()
    rows = a2.shape[0]
    if out is not None and _may_defer(done):
        parts = lib.zen_colsum_parts(rows)
        part = torch.empty(parts, cols, dtype=torch.float32, device=a.device)
        _native.check(lib.zen_colsum_partial(_native.ptr(a2), _native.ptr(part), rows, cols, _code(a2), _native.stream_ptr()),
                      "zen_colsum_partial")
        _queue_reduce(part, parts, out, accumulate, done)
        return out
    part = _scratch_buf("colsum", lib.zen_colsum_parts(rows) * cols, torch.float32, a.device)
    acc = out is not None and accumulate
    if out is None:
        out = torch.empty(cols, dtype=a.dtype, device=a.device)
    _native.check(lib.zen_colsum(_native.ptr(a2), _native.ptr(part), _native.ptr(out), rows, cols, int(acc), _code(a2),
                                 _native.stream_ptr()), "zen_colsum")
    if done is not None:
        done()
    return out


# ----------------------------------------------------------------------------- activations
def _gelu_tanh(x):
    return F.gelu(x, approximate="tanh")


def act_fwd(a: torch.Tensor, b: torch.Tensor | None, kind: str) -> torch.Tensor:
    """gelu_tanh(a) | relu(a) | silu(a) * b | gelu_tanh(a) * b.  a, b: [rows, inner] (row-strided views allowed)."""
    mode = _ACT[kind]
    if not a.is_cuda:
        af = a.float()
        if mode == 0:
            o = _gelu_tanh(af)
        elif mode == 1:
            o = F.relu(af)
        elif mode == 2:
            o = F.silu(af) * b.float()
        else:
            o = _gelu_tanh(af) * b.float()
        return o.to(a.dtype)
    inner = a.shape[-1]
    a2 = a.reshape(-1, inner) if a.dim() != 2 else a
    b2 = (b.reshape(-1, inner) if b.dim() != 2 else b) if b is not None else None
    assert a2.stride(1) == 1 and (b2 is None or b2.stride(1) == 1)
    rows = a2.shape[0]
    out = torch.empty(rows, inner, dtype=a.dtype, device=a.device)
    rc = _native.lib().zen_act_fwd(_native.ptr(a2), _native.ptr(b2), _native.ptr(out), rows, inner, a2.stride(0),
                                   b2.stride(0) if b2 is not None else inner, mode, _code(a2), _native.stream_ptr())
    _native.check(rc, "zen_act_fwd")
    return out.view(*a.shape[:-1], inner)


def act_bwd(a, b, dout, kind: str):
    """Gradients (da, db) of act_fwd; db is None for the ungated kinds."""
    mode = _ACT[kind]
    if not a.is_cuda:
        af = a.float().detach().requires_grad_(True)
        bf = b.float().detach().requires_grad_(True) if b is not None else None
        with torch.enable_grad():
            if mode == 0:
                o = _gelu_tanh(af)
            elif mode == 1:
                o = F.relu(af)
            elif mode == 2:
                o = F.silu(af) * bf
            else:
                o = _gelu_tanh(af) * bf
        gs = torch.autograd.grad(o, [af] + ([bf] if bf is not None else []), dout.float())
        return gs[0].to(a.dtype), (gs[1].to(a.dtype) if bf is not None else None)
    inner = a.shape[-1]
    a2 = a.reshape(-1, inner) if a.dim() != 2 else a
    b2 = (b.reshape(-1, inner) if b.dim() != 2 else b) if b is not None else None
    d2 = _c(dout).view(-1, inner)
    rows = a2.shape[0]
    da = torch.empty(rows, inner, dtype=a.dtype, device=a.device)
    db = torch.empty(rows, inner, dtype=a.dtype, device=a.device) if b is not None else None
    # da / db are dense [rows, inner]; the kernel strides them like a / b, so pass dense strides for outputs
    a_c = a2 if a2.stride(0) == inner else a2.contiguous()
    b_c = (b2 if b2.stride(0) == inner else b2.contiguous()) if b2 is not None else None
    rc = _native.lib().zen_act_bwd(_native.ptr(a_c), _native.ptr(b_c), _native.ptr(d2), _native.ptr(da), _native.ptr(db),
                                   rows, inner, inner, inner, mode, _code(a2), _native.stream_ptr())
    _native.check(rc, "zen_act_bwd")
    return da.view(a.shape), (db.view(a.shape) if db is not None else None)


def act_bwd_with_colsum(a: torch.Tensor, dout: torch.Tensor, kind: str):
    """(da, part) for an ungated activation on a dense CUDA [rows, inner] tensor: ``part`` holds partial column sums of
    ``da`` (fp32, one row per group of input rows) that :func:`colsum_from_parts` turns into the bias gradient of the
    layer before the activation, so that ``da`` is not read a second time for it."""
    mode = _ACT[kind]
    assert a.is_cuda and mode in (0, 1) and a.dim() == 2 and a.is_contiguous()
    rows, inner = a.shape
    d2 = _c(dout).view(rows, inner)
    lib = _native.lib()
    da = torch.empty_like(a)
    part = torch.empty(lib.zen_act_colsum_parts(rows), inner, dtype=torch.float32, device=a.device)
    _native.check(lib.zen_act_bwd_colsum(_native.ptr(a), _native.ptr(d2), _native.ptr(da), _native.ptr(part), rows, inner,
                                         mode, _code(a), _native.stream_ptr()), "zen_act_bwd_colsum")
    return da, part


def colsum_from_parts(part: torch.Tensor, out: torch.Tensor, accumulate: bool = True, done=None) -> torch.Tensor:
    """Sum the partial column sums ``part[parts, cols]`` into ``out[cols]`` (added when ``accumulate``, else written)."""
    if _may_defer(done):
        _queue_reduce(part, part.shape[0], out, accumulate, done)
        return out
    _colsum_from_parts_now(part, out, accumulate)
    if done is not None:
        done()
    return out


def _colsum_from_parts_now(part, out, accumulate):
    _native.check(_native.lib().zen_colsum_reduce(_native.ptr(part), _native.ptr(out), part.shape[0], part.shape[1],
                                                  int(accumulate), _code(out), _native.stream_ptr()), "zen_colsum_reduce")
    return out


def act_bwd_gated(x: torch.Tensor, dout: torch.Tensor, kind: str) -> torch.Tensor:
    """Gradient of the gated activation with respect to the fused [rows, 2 * inner] input (gate | up), written straight
    into one [rows, 2 * inner] tensor: the kernel reads the two halves through the row stride and stores the two
    gradients the same way, so nothing is copied or concatenated."""
    inner = x.shape[1] // 2
    if not x.is_cuda:
        da, db = act_bwd(x[:, :inner], x[:, inner:], dout, kind)
        return torch.cat([da, db], dim=1)
    assert x.dim() == 2 and x.stride(1) == 1
    d2 = _c(dout).view(-1, inner)
    rows, ld = x.shape[0], x.stride(0)
    dx = torch.empty(rows, 2 * inner, dtype=x.dtype, device=x.device)
    if ld == 2 * inner:
        rc = _native.lib().zen_act_bwd(_native.ptr(x), _native.ptr(x[:, inner:]), _native.ptr(d2), _native.ptr(dx),
                                       _native.ptr(dx[:, inner:]), rows, inner, ld, ld, _ACT[kind], _code(x),
                                       _native.stream_ptr())
        _native.check(rc, "zen_act_bwd")
        return dx
    da, db = act_bwd(x[:, :inner], x[:, inner:], dout, kind)
    dx[:, :inner].copy_(da)
    dx[:, inner:].copy_(db)
    return dx


# ----------------------------------------------------------------------------- RoPE
def rope_(x: torch.Tensor, seq: int, theta: float = 10000.0, inverse: bool = False, pos0: int = 0) -> torch.Tensor:
    """In-place rotary embedding (rotate-half) on x[tokens, heads, hd]; token t has position pos0 + t % seq."""
    tokens, heads, hd = x.shape
    if not x.is_cuda:
        half = hd // 2
        inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32) * 2 / hd))
        pos = (pos0 + torch.arange(tokens) % seq).float()
        ang = pos[:, None] * inv[None, :]
        s, c = ang.sin()[:, None, :], ang.cos()[:, None, :]
        if inverse:
            s = -s
        a, b = x[..., :half].float().clone(), x[..., half:].float().clone()
        x[..., :half] = (a * c - b * s).to(x.dtype)
        x[..., half:] = (b * c + a * s).to(x.dtype)
        return x
    assert x.stride(2) == 1 and x.stride(1) == hd
    rc = _native.lib().zen_rope(_native.ptr(x), tokens, heads, hd, x.stride(0), seq, pos0, ctypes.c_float(theta),
                                int(inverse), _code(x), _native.stream_ptr())
    _native.check(rc, "zen_rope")
    return x


# ----------------------------------------------------------------------------- embedding
def embedding_fwd(ids, wte, wpe=None, *, seq: int, pos_offset: int = 0, scale: float = 1.0):
    """out[t] = wte[ids[t]] * scale (+ wpe[pos_offset + t % seq]); ids int64 [tokens]."""
    tokens, d = ids.numel(), wte.shape[1]
    ids1 = _c(ids).view(-1)
    if not wte.is_cuda:
        out = wte[ids1]
        if scale != 1.0:
            out = (out.float() * scale).to(wte.dtype)
        if wpe is not None:
            out = (out.float() + wpe[pos_offset + torch.arange(tokens) % seq].float()).to(wte.dtype)
        return out
    out = torch.empty(tokens, d, dtype=wte.dtype, device=wte.device)
    rc = _native.lib().zen_embedding_fwd(_native.ptr(ids1), _native.ptr(wte), _native.ptr(wpe), _native.ptr(out), tokens,
                                         d, seq, pos_offset, ctypes.c_float(scale), wte.shape[0], _code(wte),
                                         _native.stream_ptr())
    _native.check(rc, "zen_embedding_fwd")
    return out


class RowSparseScratch:
    """Reusable buffers of the row-sparse embedding backward for one (vocab, d, max_rows)."""

    def __init__(self, vocab: int, d: int, max_rows: int, dtype, device):
        self.vocab, self.d, self.max_rows = vocab, d, max_rows
        self.flag = torch.zeros(vocab, dtype=torch.int32, device=device)
        self.acc = torch.zeros(max_rows, d, dtype=torch.float32, device=device)
        self.rows = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self.count = torch.zeros(1, dtype=torch.int32, device=device)
        self.vals = torch.zeros(max_rows, d, dtype=dtype, device=device)


def embedding_bwd_rows(ids, dy, vocab: int, scale: float = 1.0, scratch: RowSparseScratch | None = None):
    """Row-sparse gradient of an embedding lookup: (rows int32 ascending unique, count int32[1], vals[max_rows, d]).

    Only ``count`` leading rows are meaningful; nothing is synchronised with the host.
    """
    tokens, d = ids.numel(), dy.shape[-1]
    ids1, dy2 = _c(ids).view(-1), _c(dy).view(-1, d)
    if not dy.is_cuda:
        uniq, inv = torch.unique(ids1, return_inverse=True)
        vals = torch.zeros(uniq.numel(), d, dtype=torch.float32)
        vals.index_add_(0, inv, dy2.float() * scale)
        return uniq.to(torch.int32), torch.tensor([uniq.numel()], dtype=torch.int32), vals.to(dy.dtype)
    max_rows = min(tokens, vocab)
    if scratch is None:
        scratch = RowSparseScratch(vocab, d, max_rows, dy.dtype, dy.device)
    assert scratch.max_rows >= max_rows and scratch.vocab == vocab and scratch.d == d
    rc = _native.lib().zen_embedding_bwd_rows(_native.ptr(ids1), _native.ptr(dy2), _native.ptr(scratch.flag),
                                              _native.ptr(scratch.acc), _native.ptr(scratch.rows),
                                              _native.ptr(scratch.count), _native.ptr(scratch.vals), tokens, d, vocab,
                                              ctypes.c_float(scale), _code(dy2), _native.stream_ptr())
    _native.check(rc, "zen_embedding_bwd_rows")
    return scratch.rows, scratch.count, scratch.vals


def rows_add_(grad, rows, count, vals) -> torch.Tensor:
    """grad[rows[u]] += vals[u] for u < count (rows unique)."""
    if not grad.is_cuda:
        n = int(count.item())
        grad.index_add_(0, rows[:n].long(), vals[:n].to(grad.dtype))
        return grad
    rc = _native.lib().zen_rows_add(_native.ptr(grad), _native.ptr(rows), _native.ptr(count), _native.ptr(vals),
                                    grad.shape[1], grad.shape[0], rows.numel(), _code(grad), _native.stream_ptr())
    _native.check(rc, "zen_rows_add")
    return grad


# ----------------------------------------------------------------------------- cross entropy
def cross_entropy(logits, labels, *, grad_scale: float | None = None, ignore_index: int = -100, inplace_grad=True,
                  grad_scale_dev: torch.Tensor | None = None):
    """Per-row loss (fp32) and, when ``grad_scale`` is given, dlogits = (softmax - onehot) * grad_scale.

    With ``inplace_grad`` the gradient overwrites ``logits`` (they are not needed afterwards).
    """
    vocab = logits.shape[-1]
    lg = logits.view(-1, vocab) if logits.dim() != 2 else logits
    rows = lg.shape[0]
    lb = _c(labels).view(-1)
    if not logits.is_cuda:
        lf = lg.float()
        loss = F.cross_entropy(lf, lb, reduction="none", ignore_index=ignore_index)
        d = None
        if grad_scale is not None:
            p = torch.softmax(lf, -1)
            valid = lb != ignore_index
            onehot = torch.zeros_like(p)
            onehot[valid, lb[valid]] = 1.0
            gs = grad_scale * (float(grad_scale_dev) if grad_scale_dev is not None else 1.0)
            d = ((p - onehot) * gs * valid[:, None]).to(logits.dtype)
            if inplace_grad:
                lg.copy_(d)
                d = lg
        return loss, d
    assert lg.stride(1) == 1
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    d = None
    if grad_scale is not None:
        d = lg if inplace_grad else torch.empty_like(lg)
        assert d.stride(0) == lg.stride(0)
    rc = _native.lib().zen_xent(_native.ptr(lg), _native.ptr(lb), _native.ptr(loss), _native.ptr(d), rows, vocab,
                                lg.stride(0), ctypes.c_float(grad_scale or 0.0), _native.ptr(grad_scale_dev),
                                ctypes.c_int64(ignore_index),
                                _code(lg), _native.stream_ptr())
    _native.check(rc, "zen_xent")
    return loss, d


# ----------------------------------------------------------------------------- vocabulary-parallel cross entropy
def xent_partial(logits, labels, valid_cols: int, vocab_start: int, ignore_index: int = -100):
    """Per-row (max, sum-exp, target logit) over this rank's vocabulary shard ``logits[:, :valid_cols]``."""
    rows = logits.shape[0]
    if not logits.is_cuda:
        lf = logits[:, :valid_cols].float()
        m = lf.max(-1).values if valid_cols else torch.full((rows,), float("-inf"))
        s = (lf - m[:, None]).exp().sum(-1)
        lab = labels - vocab_start
        mine = (labels != ignore_index) & (lab >= 0) & (lab < valid_cols)
        tgt = torch.where(mine, lf.gather(1, lab.clamp(0, max(valid_cols - 1, 0))[:, None]).squeeze(1), torch.zeros(rows))
        return m, s, tgt
    m = torch.empty(rows, dtype=torch.float32, device=logits.device)
    s2 = torch.empty_like(m)
    tgt = torch.empty_like(m)
    rc = _native.lib().zen_xent_partial(_native.ptr(logits), _native.ptr(labels), _native.ptr(m), _native.ptr(s2), _native.ptr(tgt),
                                        rows, valid_cols, logits.stride(0), ctypes.c_int64(vocab_start),
                                        ctypes.c_int64(ignore_index), _code(logits), _native.stream_ptr())
    _native.check(rc, "zen_xent_partial")
    return m, s2, tgt


def xent_apply_(logits, labels, lse, valid_cols: int, vocab_start: int, grad_scale_dev=None, grad_scale: float = 1.0,
                ignore_index: int = -100):
    """In place: logits <- (exp(logits - lse) - onehot(label - vocab_start)) * scale; padding columns get zero."""
    rows, cols = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        pr = (lf - lse[:, None]).exp()
        pr[:, valid_cols:] = 0
        lab = labels - vocab_start
        mine = (labels != ignore_index) & (lab >= 0) & (lab < cols)
        pr[mine, lab[mine]] -= 1.0
        sc = grad_scale * (float(grad_scale_dev) if grad_scale_dev is not None else 1.0)
        pr = pr * sc * (labels != ignore_index)[:, None]
        logits.copy_(pr.to(logits.dtype))
        return logits
    rc = _native.lib().zen_xent_apply(_native.ptr(logits), _native.ptr(labels), _native.ptr(lse), rows, cols, valid_cols,
                                      logits.stride(0), ctypes.c_float(grad_scale), _native.ptr(grad_scale_dev),
                                      ctypes.c_int64(vocab_start), ctypes.c_int64(ignore_index), _code(logits),
                                      _native.stream_ptr())
    _native.check(rc, "zen_xent_apply")
    return logits
