"""Fused multi-tensor AdamW.

One kernel launch updates every parameter: a device-resident table lists the
tensors (parameter, optional fp32 master copy, gradient, both moments) and a
flat list of 64K-element chunks maps CTAs to tensors.  bf16 parameters keep
fp32 master weights and fp32 moments, which is what the reference gets from
ColossalAI's ``HybridAdam`` under the bf16 mixed-precision plugin
(train.py:117-123, 156).  On CPU the same update runs as plain PyTorch.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native

_CHUNK = 65536


class _AdamTensor(ctypes.Structure):
    _fields_ = [("param", ctypes.c_void_p), ("master", ctypes.c_void_p), ("grad", ctypes.c_void_p),
                ("m", ctypes.c_void_p), ("v", ctypes.c_void_p), ("numel", ctypes.c_uint64),
                ("chunk0", ctypes.c_uint64), ("wd", ctypes.c_float), ("pad", ctypes.c_float)]


class FusedAdamW(torch.optim.Optimizer):
    """AdamW with decoupled weight decay; defaults follow ``torch.optim.Adam`` / HybridAdam (wd = 0)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, master_weights=True):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.master_weights = master_weights
        self._tables: dict = {}
        self._step = 0
        self._step_dev = None          # device step counter, used when the step is captured in a CUDA graph

    def _init_state(self, p):
        st = self.state[p]
        if not st:
            st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
            if self.master_weights and p.dtype != torch.float32:
                st["master"] = p.detach().float().clone()
        return st

    def _table_for(self, gi, group, params):
        """Device table for one (group, dtype); rebuilt when any pointer changes."""
        key = tuple((p.data_ptr(), p.grad.data_ptr()) for p in params)
        cached = self._tables.get((gi, params[0].dtype))
        if cached and cached[0] == key:
            return cached[1:]
        lib = _native.lib()
        assert lib.zen_adam_tensor_size() == ctypes.sizeof(_AdamTensor)
        arr = (_AdamTensor * len(params))()
        chunk_tensor = []
        c0 = 0
        for i, p in enumerate(params):
            st = self._init_state(p)
            n = p.numel()
            assert p.is_contiguous() and p.grad.is_contiguous() and p.data_ptr() % 16 == 0 and p.grad.data_ptr() % 16 == 0
            arr[i] = _AdamTensor(p.data_ptr(), st["master"].data_ptr() if "master" in st else 0, p.grad.data_ptr(),
                                 st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr(), n, c0,
                                 group["weight_decay"], 0.0)
            nch = (n + _CHUNK - 1) // _CHUNK
            chunk_tensor.extend([i] * nch)
            c0 += nch
        raw = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).clone()
        table = raw.to(params[0].device)
        ct = torch.tensor(chunk_tensor, dtype=torch.int32, device=params[0].device)
        self._tables[(gi, params[0].dtype)] = (key, table, ct, c0)
        return table, ct, c0

    def enable_device_step(self, device):
        """Keep the step count on the device so that ``step`` can be captured in a CUDA graph and replayed."""
        self._step_dev = torch.full((1,), self._step, dtype=torch.int32, device=device)

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        self._step += 1
        t = self._step
        if self._step_dev is not None:
            self._step_dev += 1
        for gi, group in enumerate(self.param_groups):
            b1, b2 = group["betas"]
            lr, eps, wd = group["lr"], group["eps"], group["weight_decay"]
            bc1, bc2 = 1.0 - b1 ** t, 1.0 - b2 ** t
            live = [p for p in group["params"] if p.grad is not None]
            if not live:
                continue
            if live[0].is_cuda:
                by_dtype: dict = {}
                for p in live:
                    by_dtype.setdefault(p.dtype, []).append(p)
                for dtype, ps in by_dtype.items():
                    table, ct, nch = self._table_for(gi, group, ps)
                    rc = _native.lib().zen_adamw(_native.ptr(table), len(ps), _native.ptr(ct), ctypes.c_uint64(nch),
                                                 ctypes.c_float(lr), ctypes.c_float(b1), ctypes.c_float(b2),
                                                 ctypes.c_float(eps), ctypes.c_float(bc1), ctypes.c_float(bc2),
                                                 ctypes.c_float(grad_scale), _native.ptr(self._step_dev),
                                                 _native.DTYPE_CODE[dtype],
                                                 _native.stream_ptr())
                    _native.check(rc, "zen_adamw")
            else:
                for p in live:
                    st = self._init_state(p)
                    g = p.grad.float() * grad_scale
                    st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
                    st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                    w = st["master"] if "master" in st else p.data.float()
                    den = (st["exp_avg_sq"] / bc2).sqrt_().add_(eps)
                    w = w * (1 - lr * wd) - lr * (st["exp_avg"] / bc1) / den
                    if "master" in st:
                        st["master"].copy_(w)
                    p.data.copy_(w.to(p.dtype))
        return None

    @property
    def steps_done(self) -> int:
        """Optimizer steps taken so far.  With the device counter enabled that counter is the truth: a replayed CUDA
        graph advances it without running the host side of ``step`` (reading it synchronises the device)."""
        if self._step_dev is not None:
            self._step = int(self._step_dev.item())
        return self._step

    def state_dict(self):
        sd = super().state_dict()
        sd["zen_step"] = self.steps_done
        return sd

    def load_state_dict(self, sd):
        sd = dict(sd)
        self._step = sd.pop("zen_step", 0)
        # torch's loader casts floating-point state to the parameter's dtype, which would turn the fp32 moments and
        # master weights of a bf16 parameter into bf16 (the kernel reads them as fp32): load the groups through torch,
        # the per-parameter state here, dtype kept
        saved = sd.get("state", {})
        super().load_state_dict({"state": {}, "param_groups": sd["param_groups"]})
        ids = [i for g in sd["param_groups"] for i in g["params"]]
        params = [p for g in self.param_groups for p in g["params"]]
        for i, p in zip(ids, params):
            if i in saved:
                self.state[p] = {k: (v.detach().clone().to(p.device) if torch.is_tensor(v) else v) for k, v in saved[i].items()}
        self._tables.clear()
        if self._step_dev is not None:           # the bias corrections of a captured step read the device counter
            self._step_dev.fill_(self._step)
