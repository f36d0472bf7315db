"""NVTX ranges and device-side stage timers.

``trace_range(name)`` is a context manager that pushes an NVTX range when tracing is enabled
(``enable_tracing(True)`` or ``ZEN_TRACE=1``) and costs one branch otherwise.  Range names follow the
reference's annotations (train.py:65-69,176,199-209; comm.py:66-144; tensor_load_balance.py:25-44) so
that Nsight Systems timelines of both line up.  ``StageTimer`` records CUDA events around stages and
reports device milliseconds.
"""
from __future__ import annotations

import contextlib
import os

import torch

_ENABLED = os.environ.get("ZEN_TRACE", "0") == "1"


def enable_tracing(on: bool = True) -> None:
    global _ENABLED
    _ENABLED = on


def tracing_enabled() -> bool:
    return _ENABLED


@contextlib.contextmanager
def trace_range(name: str):
    if _ENABLED and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class StageTimer:
    """CUDA-event timer: ``with timer.stage("x"): ...`` then ``timer.results()`` -> {name: ms} (synchronises)."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self._events: list = []

    @contextlib.contextmanager
    def stage(self, name: str):
        if not self.enabled:
            yield
            return
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        try:
            with trace_range(name):
                yield
        finally:
            e.record()
            self._events.append((name, s, e))

    def results(self) -> dict:
        if not self.enabled:
            return {}
        torch.cuda.synchronize()
        out: dict = {}
        for name, s, e in self._events:
            out[name] = out.get(name, 0.0) + s.elapsed_time(e)
        self._events.clear()
        return out
