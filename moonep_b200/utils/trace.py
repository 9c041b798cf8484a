"""Lightweight tracing: named spans timed with CUDA events on the current stream, mirrored as
NVTX ranges for Nsight.  The reference has no tracing layer (its authors profile by hand and
only expose ``--no-graph`` switches, benchmarks/bench_prefetch.py:235-236); here any code path can
be wrapped in ``with tracer.span("name")`` at no cost when tracing is off.

Usage::

    tracer = Tracer(enabled=True)
    with tracer.span("dispatch"):
        ...
    print(tracer.summary())          # mean / total ms per span name (synchronises)
"""
from __future__ import annotations

import contextlib
from collections import OrderedDict

import torch


class Tracer:
    def __init__(self, enabled: bool = False, nvtx: bool = True):
        self.enabled = enabled
        self.nvtx = nvtx
        self._spans: list[tuple[str, torch.cuda.Event, torch.cuda.Event]] = []

    @contextlib.contextmanager
    def span(self, name: str):
        if not self.enabled:
            yield
            return
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            if self.nvtx:
                torch.cuda.nvtx.range_pop()
            self._spans.append((name, a, b))

    def reset(self) -> None:
        self._spans.clear()

    def summary(self) -> "OrderedDict[str, dict]":
        """Per span name: calls, total ms, mean ms (device time between the span's events)."""
        torch.cuda.synchronize()
        out: "OrderedDict[str, dict]" = OrderedDict()
        for name, a, b in self._spans:
            d = out.setdefault(name, {"calls": 0, "total_ms": 0.0})
            d["calls"] += 1
            d["total_ms"] += a.elapsed_time(b)
        for d in out.values():
            d["mean_ms"] = d["total_ms"] / d["calls"]
        return out


NULL_TRACER = Tracer(enabled=False)
