"""Timers.  ``LocalTimer`` is the reference's host timer (synchronise + wall clock at both ends,
reference: train.py:397-423).  ``DeviceTimer`` times a region with CUDA events on the current
stream and reports the maximum over ranks, which is what throughput numbers are quoted on."""
from __future__ import annotations

import time

import torch

from .dist import all_reduce_max


class LocalTimer:
    def __init__(self, device: torch.device):
        if device.type == "cuda":
            self.synchronize = lambda: torch.cuda.synchronize(device=device)
        else:
            self.synchronize = lambda: None
        self.measurements: list[float] = []
        self.start_time = None

    def __enter__(self):
        self.synchronize()
        self.start_time = time.time()
        return self

    def __exit__(self, exc_type, value, traceback):
        if traceback is None:
            self.synchronize()
            self.measurements.append(time.time() - self.start_time)
        self.start_time = None

    def avg_elapsed_ms(self) -> float:
        if not self.measurements:
            return 0.0
        return 1000 * (sum(self.measurements) / len(self.measurements))

    def reset(self):
        self.measurements = []
        self.start_time = None


class DeviceTimer:
    """``with DeviceTimer(device) as t: ...`` then ``t.ms`` (this rank) / ``t.max_ms()`` (all ranks)."""

    def __init__(self, device: torch.device):
        self.device = device
        self.ms = 0.0
        self._cuda = device.type == "cuda"

    def __enter__(self):
        if self._cuda:
            torch.cuda.synchronize(self.device)
            self._start = torch.cuda.Event(enable_timing=True)
            self._end = torch.cuda.Event(enable_timing=True)
            self._start.record()
        else:
            self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self._cuda:
            self._end.record()
            torch.cuda.synchronize(self.device)
            self.ms = self._start.elapsed_time(self._end)
        else:
            self.ms = 1000 * (time.perf_counter() - self._t0)

    def max_ms(self) -> float:
        return all_reduce_max(self.ms, self.device)
