"""Data-parallel gradient reducer with bucketed, overlapped communication and DDP-style comm hooks.

``ZenDDP`` wraps a module the way ``torch.nn.parallel.DistributedDataParallel`` does for the
reference (through ColossalAI's plugin, train.py:157,184-185): parameters are packed into flat
buckets of ``bucket_cap_mb`` in reverse registration order, ``param.grad`` are views of those buffers,
a bucket's communication starts as soon as its last gradient has been accumulated, on a side stream
that waits for the producing stream, and ``finalize_grads()`` joins everything before the optimizer
step.  ``register_comm_hook(state, hook)`` takes hooks with torch's signature
``hook(state, bucket) -> Future[Tensor]``; the default is an averaged dense all-reduce.
Parameters flagged ``zen_sparse_only`` (an untied embedding whose gradient exists only as sparse rows)
stay out of the buckets and are filled by the embedding row synchroniser.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..utils.trace import trace_range


class GradBucket:
    """The part of ``torch.distributed.GradBucket`` that hooks use."""

    def __init__(self, index: int, buffer: torch.Tensor, params: list, last: bool):
        self._index, self._buffer, self._params, self._last = index, buffer, params, last

    def index(self) -> int:
        return self._index

    def buffer(self) -> torch.Tensor:
        return self._buffer

    def set_buffer(self, t: torch.Tensor) -> None:
        self._buffer.copy_(t)

    def is_last(self) -> bool:
        return self._last

    def parameters(self) -> list:
        return list(self._params)

    def gradients(self) -> list:
        return [p.grad for p in self._params]


class _Bucket:
    def __init__(self, index, params, dtype, device, storage=None):
        self.index, self.params = index, params
        sizes = [(p.numel() + 7) // 8 * 8 for p in params]          # 16-byte aligned views for bf16
        self.numel = sum(sizes)
        self.arena_off = None                                        # byte offset in the multicast arena, when it lives there
        self.buffer = storage if storage is not None else torch.zeros(self.numel, dtype=dtype, device=device)
        self.views, off = [], 0
        for p, s in zip(params, sizes):
            self.views.append(self.buffer[off:off + p.numel()].view(p.shape))
            off += s
        self.pending = len(params)
        self.future = None
        self.launched = False


class ZenDDP(nn.Module):
    def __init__(self, module: nn.Module, process_group=None, bucket_cap_mb: float = 25.0, embedding_sync=None,
                 overlap: bool = True, dense_transport: str = "nccl"):
        super().__init__()
        self.module = module
        self.process_group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.embedding_sync = embedding_sync
        self._hook, self._hook_state = None, None
        params = [p for p in module.parameters() if p.requires_grad]
        self.device = params[0].device
        self._sparse_only = [p for p in params if getattr(p, "zen_sparse_only", False)]
        dense = [p for p in params if not getattr(p, "zen_sparse_only", False)]
        cap = int(bucket_cap_mb * 1024 * 1024)
        self.buckets: list[_Bucket] = []
        # A parameter flagged ``zen_early`` gets its whole gradient at the very start of backward (the tied token
        # embedding when its lookup rows travel through the row-sparse path: what is left is the LM-head product).  It
        # leads the bucket order in a bucket of its own, so its all-reduce overlaps the rest of backward instead of
        # waiting at the end with the first layers' parameters.
        early = [p for p in dense if getattr(p, "zen_early", False)]
        groups: list[tuple[list, torch.dtype]] = [([p], p.dtype) for p in early]
        cur, cur_bytes, cur_dtype = [], 0, None
        for p in reversed(dense):
            if getattr(p, "zen_early", False):
                continue
            nbytes = p.numel() * p.element_size()
            if cur and (cur_bytes + nbytes > cap or p.dtype != cur_dtype):
                groups.append((cur, cur_dtype))
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            cur_dtype = p.dtype
        if cur:
            groups.append((cur, cur_dtype))
        # "nvls": the buckets live in one multicast-mapped symmetric region and are reduced through the NVSwitch by this
        # library's own kernel on a few CTAs; otherwise plain device memory and the library all-reduce
        self.arena = None
        if (dense_transport == "nvls" and self.world > 1 and self.device.type == "cuda"
                and all(dt in (torch.bfloat16, torch.float32) for _, dt in groups)):
            from .nvls_allreduce import MulticastArena

            sizes = [sum((p.numel() + 7) // 8 * 8 for p in ps) * torch.empty(0, dtype=dt).element_size() for ps, dt in groups]
            offs, off = [], 0
            for sz in sizes:
                offs.append(off)
                off += (sz + 255) // 256 * 256
            try:
                self.arena = MulticastArena(off, process_group)
            except Exception as ex:                               # no multicast on this fabric: keep the library path
                self.arena, self.arena_error = None, f"{type(ex).__name__}: {ex}"
        for i, (ps, dt) in enumerate(groups):
            storage = None
            if self.arena is not None:
                storage = self.arena.view(offs[i], sum((p.numel() + 7) // 8 * 8 for p in ps), dt)
            b = _Bucket(len(self.buckets), ps, dt, self.device, storage)
            if self.arena is not None:
                b.arena_off = offs[i]
            self.buckets.append(b)
        self._bucket_of, self._view_of = {}, {}
        for b in self.buckets:
            for p, v in zip(b.params, b.views):
                p.grad = v
                self._bucket_of[id(p)] = b
                self._view_of[id(p)] = v
                p.register_post_accumulate_grad_hook(self._on_autograd_ready)
                # ops that can add their result into the bucket view themselves do so and call zen_ready
                p.zen_direct_grad = True
                p.zen_ready = self._on_grad_ready
        for p in self._sparse_only:
            p.grad = torch.zeros_like(p)
        self._cuda = self.device.type == "cuda"
        self.comm_stream = torch.cuda.Stream() if (self._cuda and overlap) else None
        self._launched = 0
        self._nccl = self.world > 1 and self._cuda and dist.get_backend(process_group) == "nccl"
        self.require_sync = True
        self.timeline = None             # set to a list to collect per-step CUDA events (see exposed_comm_us)

    def exposed_comm_us(self) -> list[dict]:
        """Per recorded step (``timeline = []`` switches recording on; eager steps only): microseconds between the end of
        backward on the compute stream and the end of the bucket communication on the side stream (the part of the
        dense synchronisation that backward did not hide), and up to the end of the row-sparse embedding exchange."""
        torch.cuda.synchronize()
        out = []
        for a, b, c in self.timeline or []:
            out.append({"dense_exposed_us": max(0.0, a.elapsed_time(b) * 1e3), "sync_exposed_us": max(0.0, a.elapsed_time(c) * 1e3)})
        return out

    # ---- torch DDP surface --------------------------------------------------------------------
    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    def register_comm_hook(self, state, hook) -> None:
        self._hook_state, self._hook = state, hook

    def no_sync(self):
        ddp = self

        class _Ctx:
            def __enter__(self_):
                ddp.require_sync = False

            def __exit__(self_, *exc):
                ddp.require_sync = True

        return _Ctx()

    # ---- reduction --------------------------------------------------------------------------------
    def _default_hook(self, _state, bucket: GradBucket):
        buf = bucket.buffer()
        b = self.buckets[bucket.index()]
        if self.world > 1 and self.arena is not None and b.arena_off is not None and buf.data_ptr() == b.buffer.data_ptr():
            self.arena.allreduce_(b.arena_off, b.numel * buf.element_size(), buf.dtype, 1.0 / self.world)
        elif self.world > 1:
            if self._nccl:
                dist.all_reduce(buf, op=dist.ReduceOp.AVG, group=self.process_group)   # the mean inside the collective
            else:
                buf.div_(self.world)
                dist.all_reduce(buf, group=self.process_group)
        from .hooks import _Ready

        return _Ready(buf)

    def _on_autograd_ready(self, p):
        p.zen_autograd_done = True
        self._on_grad_ready(p, from_autograd=True)

    def _on_grad_ready(self, p, from_autograd: bool = False):
        """A gradient contribution for ``p`` has landed in its bucket view.  A parameter is complete when every
        op that claimed a direct write has signalled and, if an autograd-path use was declared (or happened), the
        accumulate-grad hook has fired; its bucket goes out when all its parameters are complete."""
        b = self._bucket_of[id(p)]
        v = self._view_of[id(p)]
        if p.grad.data_ptr() != v.data_ptr():
            # autograd replaced the view (first accumulation into an undefined grad): copy back in
            v.copy_(p.grad)
            p.grad = v
        if not from_autograd:
            p.zen_signals = getattr(p, "zen_signals", 0) + 1
        done_direct = getattr(p, "zen_signals", 0) == getattr(p, "zen_expected", 0)
        done_auto = getattr(p, "zen_autograd_done", False) or not getattr(p, "zen_autograd_use", False)
        if done_direct and done_auto and not getattr(p, "zen_complete", False):
            p.zen_complete = True
            b.pending -= 1
            if b.pending == 0 and self.require_sync and not b.launched:
                self._launch(b)

    def _launch(self, b: _Bucket):
        hook = self._hook or self._default_hook
        b.launched = True
        if self._hook is None and self.world == 1:
            b.future = None
            return
        gb = GradBucket(b.index, b.buffer, b.params, b.index == len(self.buckets) - 1)
        with trace_range(f"bucket{b.index}"):
            if self.comm_stream is not None:
                self.comm_stream.wait_stream(torch.cuda.current_stream())
                self._comm_used = True
                with torch.cuda.stream(self.comm_stream):
                    b.future = hook(self._hook_state, gb)
            else:
                b.future = hook(self._hook_state, gb)
        self._launched += 1

    def finalize_grads(self) -> None:
        """Join all bucket communication, write hook results back, then apply the sparse embedding rows."""
        from ..ops import gemm as _gemm

        _gemm.flush_deferred()               # weight gradients still queued for a grouped launch (normally none here)
        if self.require_sync:
            for b in self.buckets:
                if not b.launched:           # parameters without a gradient this step, or undeclared uses
                    for p, v in zip(b.params, b.views):
                        if getattr(p, "zen_fresh", False) and getattr(p, "zen_stale", False):
                            v.zero_()        # nobody wrote it: do not send (or apply) the last step's gradient again
                            p.zen_stale = False
                    self._launch(b)
            used = self.comm_stream is not None and getattr(self, "_comm_used", False)
            ctx = torch.cuda.stream(self.comm_stream) if used else _null()
            with ctx:
                for b in self.buckets:
                    if b.future is not None:
                        res = b.future.wait() if hasattr(b.future, "wait") else b.future
                        if isinstance(res, (list, tuple)):
                            res = res[0]
                        if res is not b.buffer and res.data_ptr() != b.buffer.data_ptr():
                            b.buffer.copy_(res.reshape(-1))
                        b.future = None
            if used:                      # join only a stream that was forked from this one during the step
                if self.timeline is not None:
                    # backward has been enqueued up to here; what the communication stream still has to do after this
                    # point is the exposed (not overlapped) part of the gradient synchronisation
                    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
                    ev[0].record(torch.cuda.current_stream())
                    ev[1].record(self.comm_stream)
                    self._timeline_pending = ev
                torch.cuda.current_stream().wait_stream(self.comm_stream)
                self._comm_used = False
            if hasattr(self.module, "sync_replicated_grads"):
                self.module.sync_replicated_grads()
            if self.embedding_sync is not None:
                emb = self.embedding_sync
                target = emb.target_param
                emb.sync_into(target.grad, zero_first=getattr(target, "zen_sparse_only", False))
            if self.timeline is not None and getattr(self, "_timeline_pending", None) is not None:
                ev = self._timeline_pending
                ev[2].record(torch.cuda.current_stream())          # after the row synchronisation as well
                self.timeline.append(ev)
                self._timeline_pending = None
        for b in self.buckets:
            b.pending = len(b.params)
            b.launched = False
            for p in b.params:
                p.zen_direct_only = (getattr(p, "zen_expected", 0) > 0 and not getattr(p, "zen_autograd_use", False)
                                     and not getattr(p, "zen_autograd_done", False) and getattr(p, "zen_complete", False))
                p.zen_signals = 0
                p.zen_expected = 0
                p.zen_autograd_use = False
                p.zen_autograd_done = False
                p.zen_complete = False

    def zero_grad(self, set_to_none: bool = False) -> None:
        """Arm the next step.  A parameter whose gradient came only from direct writers in the step that just ended
        is not zeroed: its first writer of the next step overwrites the view (``zen_fresh``).  The others (gradients
        that autograd accumulates) are zeroed."""
        for b in self.buckets:
            lazy = [bool(getattr(p, "zen_direct_only", False)) for p in b.params]
            if not any(lazy):
                b.buffer.zero_()
            elif not all(lazy):
                for p, v, l in zip(b.params, b.views, lazy):
                    if not l:
                        v.zero_()
            for p, l in zip(b.params, lazy):
                p.zen_fresh = True              # nothing written yet in the coming step: the first direct writer overwrites
                p.zen_stale = l                 # ... and the view still holds the old gradient
        # gradients of row-sparse-only parameters are rebuilt from zero by the embedding sync of the next step


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
