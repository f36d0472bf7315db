"""Row-sparse synchronisation of the token-embedding gradient across data-parallel ranks.

The embedding backward hands over (unique rows, count, summed gradient rows) instead of scattering
into a dense [V, d] tensor.  After backward those rows are summed across the DP group with the
row-granule sparse all-reduce (P2P stores over NVLink on GPU, an all-gather on CPU/gloo) and added into
the dense gradient that the optimizer reads.  For tied embeddings the dense part of that gradient (the
LM-head product) travels through the ordinary dense bucket all-reduce; an untied embedding has no
dense part and its gradient buffer is zero-filled first.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import elementwise as E


class EmbeddingRowSync:
    def __init__(self, vocab: int, d: int, max_tokens: int, dp_group=None, dtype=torch.bfloat16, device=None,
                 mean: bool = True, deterministic: bool = False):
        self.vocab, self.d, self.group, self.dtype = vocab, d, dp_group, dtype
        self.P = dist.get_world_size(dp_group) if dist.is_initialized() else 1
        self.scale = 1.0 / self.P if mean else 1.0
        self.max_rows = min(max_tokens, vocab)
        self.device = torch.device(device) if device is not None else None
        self._scratch = None
        self._engine = None
        self._pending = None
        self.deterministic = deterministic
        self.last_count = None
        self.wait_ms = 30000.0         # bound of every wait on a peer (training: generous; tests construct engines with short ones)
        self.early = True              # start the row exchange from ``put`` (on a side stream) instead of from ``sync_into``
        self._stream = None
        self._started = False
        self.force_library = False     # set after a reported failure of the peer-memory engine: all-gather the rows instead

    # ---- called from EmbeddingFn.backward -----------------------------------------------------
    def scratch_for(self, tokens: int, dy: torch.Tensor):
        if not dy.is_cuda:
            return None
        if self._scratch is None:
            self._scratch = E.RowSparseScratch(self.vocab, self.d, self.max_rows, dy.dtype, dy.device)
        return self._scratch

    def put(self, rows, count, vals):
        if self._pending is not None:
            raise RuntimeError("a row-sparse gradient is already pending (gradient accumulation over several "
                               "micro-batches must call sync between them)")
        self._pending = (rows, count, vals)
        if self.early and self._engine is not None and not self.force_library and vals.is_cuda:
            # the rows exist as soon as the embedding backward has run: exchange them on a side stream now, while the
            # last dense buckets are still in flight; only the final add into the gradient waits for the dense sync
            if self._stream is None:
                self._stream = torch.cuda.Stream()
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                self._engine.start(rows, count, vals)
            self._started = True

    # ---- called by the reducer after backward ---------------------------------------------------
    def prepare(self, device):
        """Allocate the symmetric buffers (collective) ahead of the first step."""
        if self.P > 1 and device.type == "cuda" and self._engine is None:
            from ..sparse.row_engine import RowSparseAllReduce

            self._engine = RowSparseAllReduce(self.vocab, self.d, self.max_rows, self.group, dtype=self.dtype,
                                              deterministic=self.deterministic, wait_ms=self.wait_ms)

    def sync_into(self, grad: torch.Tensor, zero_first: bool = False):
        if self._pending is None:
            if zero_first:
                grad.zero_()
            return grad
        rows, count, vals = self._pending
        self._pending = None
        self.last_count = count
        if zero_first:
            grad.zero_()
        if self.P == 1:
            E.rows_add_(grad, rows, count, vals)
            return grad
        if self._started:
            self._started = False
            torch.cuda.current_stream().wait_stream(self._stream)
            self._engine.finish(grad, scale=self.scale)
        elif grad.is_cuda and not self.force_library:
            self.prepare(grad.device)
            self._engine(rows, count, vals, grad, scale=self.scale)
        else:
            from ..sparse.row_engine import dist_rows_allreduce

            dist_rows_allreduce(rows, count, vals, grad, self.group, self.scale)
        return grad

    def check(self) -> int:
        return self._engine.check() if self._engine is not None else 0
