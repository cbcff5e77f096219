"""Device-side timers.  The reference times its four training phases with a host clock between two
full device synchronisations each (eight syncs per step; reference: train.py:397-423).  Here a
phase is bracketed by two CUDA events on the current stream and nothing waits: the events are read
when the numbers are wanted (every ``--log-freq`` steps), so timing costs no synchronisation inside
the step.  Throughput is quoted on the maximum over ranks."""
from __future__ import annotations

import time

import torch

from .dist import all_reduce_max


class PhaseTimer:
    """``with timer: ...`` records one interval; ``avg_elapsed_ms()`` averages the recorded ones
    (synchronising on their last event), ``reset()`` forgets them."""

    def __init__(self, device: torch.device):
        self.device = device
        self._cuda = device.type == "cuda"
        self._pairs: list = []
        self._host_ms: list = []
        self._open = None

    def __enter__(self):
        if self._cuda:
            start = torch.cuda.Event(enable_timing=True)
            start.record(torch.cuda.current_stream(self.device))
            self._open = start
        else:
            self._open = time.perf_counter()
        return self

    def __exit__(self, exc_type, value, traceback):
        if traceback is None and self._open is not None:
            if self._cuda:
                end = torch.cuda.Event(enable_timing=True)
                end.record(torch.cuda.current_stream(self.device))
                self._pairs.append((self._open, end))
            else:
                self._host_ms.append(1000 * (time.perf_counter() - self._open))
        self._open = None

    def avg_elapsed_ms(self) -> float:
        if self._cuda:
            if not self._pairs:
                return 0.0
            self._pairs[-1][1].synchronize()
            return sum(a.elapsed_time(b) for a, b in self._pairs) / len(self._pairs)
        return sum(self._host_ms) / len(self._host_ms) if self._host_ms else 0.0

    def reset(self) -> None:
        self._pairs, self._host_ms, self._open = [], [], None


def max_over_ranks(ms: float, device: torch.device) -> float:
    """The slowest rank sets the pace: MAX over ranks of a per-rank time."""
    return all_reduce_max(ms, device)
