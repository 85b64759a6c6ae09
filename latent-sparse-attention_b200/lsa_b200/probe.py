"""Named regions a timing harness can record, free when nobody listens.

The reference marks its selector's stages the same way (`probe.region`, src/lsa/sglang/index/probe.py:1-31): a region
is a null context unless a recorder is installed. `CudaEventRecorder` brackets each region with CUDA events on the
current stream, so a benchmark reads per-stage device time without synchronising inside the step.
"""

from __future__ import annotations

import contextlib
from collections import defaultdict

import torch

_recorder = None


def install(recorder) -> None:
    global _recorder
    _recorder = recorder


def uninstall() -> None:
    install(None)


def region(name: str):
    if _recorder is None:
        return contextlib.nullcontext()
    return _recorder.region(name)


class CudaEventRecorder:
    """Collects (start, stop) event pairs per region name; `totals_ms()` synchronises and sums them."""

    def __init__(self) -> None:
        self.events = defaultdict(list)

    @contextlib.contextmanager
    def region(self, name: str):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        try:
            yield
        finally:
            stop.record()
            self.events[name].append((start, stop))

    def clear(self) -> None:
        self.events.clear()

    def totals_ms(self) -> dict:
        torch.cuda.synchronize()
        return {name: (sum(a.elapsed_time(b) for a, b in pairs), len(pairs)) for name, pairs in self.events.items()}
