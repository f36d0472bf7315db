"""Seeded synthetic token streams with a Zipf(s) law over the vocabulary.

Token id ``k`` (0-based) has probability proportional to ``1 / (k + 1) ** s``, so the embedding rows
touched by a batch are a small, skewed subset of the table -- the regime the sparse embedding
synchronisation is built for.  Batches are produced on the host in pinned memory; the cursor (step
counter) is part of the checkpoint so that a resumed run sees the same stream.  The reference reads
RedPajama through HuggingFace ``datasets`` (utils.py:11-31); that needs the network, so ``--data hf``
is optional in ``train.py`` and synthetic data is the default.
"""
from __future__ import annotations

import torch


def zipf_cdf(vocab: int, s: float) -> torch.Tensor:
    w = 1.0 / torch.arange(1, vocab + 1, dtype=torch.float64) ** s
    return torch.cumsum(w / w.sum(), 0)


class ZipfTokenStream:
    """Infinite iterator of ``{"input_ids", "labels"}`` int64 [batch, seq] pinned host tensors for one DP rank."""

    def __init__(self, vocab: int, seq: int, batch: int, s: float = 1.1, seed: int = 0, dp_rank: int = 0,
                 pin: bool = True, pool: int = 0):
        self.vocab, self.seq, self.batch, self.s, self.seed, self.dp_rank = vocab, seq, batch, s, seed, dp_rank
        self.cdf = zipf_cdf(vocab, s)
        self.step = 0
        self.pin = pin and torch.cuda.is_available()
        self._pool = [self._make(i) for i in range(pool)] if pool else None

    def _make(self, step: int) -> dict:
        g = torch.Generator().manual_seed((self.seed * 1_000_003 + self.dp_rank) * 1_000_003 + step)
        u = torch.rand(self.batch * self.seq, generator=g, dtype=torch.float64)
        ids = torch.searchsorted(self.cdf, u).clamp_(max=self.vocab - 1).view(self.batch, self.seq)
        if self.pin:
            ids = ids.pin_memory()
        return {"input_ids": ids, "labels": ids}

    def __iter__(self):
        return self

    def __next__(self) -> dict:
        b = self._pool[self.step % len(self._pool)] if self._pool else self._make(self.step)
        self.step += 1
        return b

    def state_dict(self) -> dict:
        return {"step": self.step, "seed": self.seed, "dp_rank": self.dp_rank}

    def load_state_dict(self, sd: dict) -> None:
        self.step = int(sd["step"])

    def row_density(self, nbatches: int = 4) -> float:
        """Mean fraction of vocabulary rows touched by one batch."""
        tot = 0.0
        for i in range(nbatches):
            tot += self._make(10_000 + i)["input_ids"].unique().numel() / self.vocab
        return tot / nbatches
