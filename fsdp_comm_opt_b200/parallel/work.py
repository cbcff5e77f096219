"""``AggregatedWork``: one ``dist.Work`` that stands for several child collectives plus a
post-processing step (decode, dequantise) that must run exactly once after them.

Same constructor and the same eight methods as the reference class
(reference: main/work.py:6-89).  Behavioural differences:

* ``wait(None)`` works.  The reference forwards ``None`` to the child ``Work.wait`` and pybind
  rejects it (main/work.py:53-56), which breaks FSDP2's async unshard path.
* ``wait()`` on CUDA makes the *current stream* wait for the post-processing event instead of
  blocking the host (c10d semantics); the host blocks only when a timeout is given or when the
  work is CPU-only.  ``synchronize()`` is the explicit host-blocking form.
* an optional ``status_fn`` is polled after completion so that a device-side bounded wait that
  gave up (fused symmetric-memory kernels) surfaces as a Python exception.
* an optional ``ready_event`` (recorded by the caller on the stream that launched the device work)
  ties the Work to that stream: ``wait`` / ``block_current_stream`` make the *current* stream wait
  for it and ``is_completed`` reports ``event.query()``, so a caller on another stream is ordered
  after a collective that is one kernel launch with no child ``Work`` at all.
"""
from __future__ import annotations

import threading
from datetime import timedelta
from typing import Callable, Iterable, Optional

import torch
import torch.distributed as dist


class AggregatedWork(dist.Work):
    def __init__(self, works: Iterable[dist.Work], postprocess_fn: Optional[Callable[[], None]] = None,
                 *, status_fn: Optional[Callable[[], None]] = None,
                 ready_event: Optional["torch.cuda.Event"] = None):
        super().__init__()
        self.ready_event = ready_event
        self.works = [w for w in works if w is not None]
        self.postprocess_fn = postprocess_fn
        self.status_fn = status_fn
        self._done = False
        self._exception: Optional[BaseException] = None
        self._lock = threading.Lock()
        self._event: Optional[torch.cuda.Event] = None

    # -- internals ---------------------------------------------------------------------------
    def _run_postprocess_once(self) -> None:
        with self._lock:
            if self._done:
                return
            if self._exception is not None:
                raise self._exception
            try:
                if self.postprocess_fn is not None:
                    self.postprocess_fn()
                if torch.cuda.is_available() and torch.cuda.is_initialized():
                    self._event = torch.cuda.Event()
                    self._event.record(torch.cuda.current_stream())
            except BaseException as e:  # remembered so every later wait() re-raises it
                self._exception = e
                raise
            self._done = True

    @staticmethod
    def _child_wait(w: dist.Work, timeout: Optional[timedelta]) -> None:
        if timeout is None:
            w.wait()
        else:
            w.wait(timeout)

    # -- dist.Work surface -------------------------------------------------------------------
    def is_completed(self) -> bool:
        if self._exception is not None:
            return True
        if not all(w.is_completed() for w in self.works):
            return False
        if self.ready_event is not None and not self.ready_event.query():
            return False
        try:
            self._run_postprocess_once()
        except BaseException:
            return True
        return True

    def is_success(self) -> bool:
        try:
            self.wait()
            return self._exception is None
        except Exception:
            return False

    def exception(self):
        return self._exception

    def wait(self, timeout: Optional[timedelta] = None) -> bool:
        if self._exception is not None:
            raise self._exception
        try:
            for w in self.works:
                self._child_wait(w, timeout)
            if self.ready_event is not None:
                if timeout is not None:
                    self.ready_event.synchronize()
                else:
                    torch.cuda.current_stream().wait_event(self.ready_event)
            self._run_postprocess_once()
            if self._event is not None:
                if timeout is not None:
                    self._event.synchronize()
                else:
                    torch.cuda.current_stream().wait_event(self._event)
            if self.status_fn is not None:
                self.status_fn()
            return True
        except BaseException as e:
            self._exception = e
            raise

    def synchronize(self) -> None:
        """Host-blocking wait (what the reference's ``wait`` did)."""
        self.wait()
        if self.ready_event is not None:
            self.ready_event.synchronize()
        if self._event is not None:
            self._event.synchronize()

    def block_current_stream(self) -> None:
        for w in self.works:
            if hasattr(w, "block_current_stream"):
                w.block_current_stream()
            else:
                w.wait()
        if self.ready_event is not None:
            torch.cuda.current_stream().wait_event(self.ready_event)
        self._run_postprocess_once()
        if self._event is not None:
            torch.cuda.current_stream().wait_event(self._event)

    def get_future(self) -> torch.futures.Future:
        futs = [w.get_future() for w in self.works]
        if not futs:
            fut: torch.futures.Future = torch.futures.Future()
            self._run_postprocess_once()
            fut.set_result([])
            return fut

        def _then(done):
            self._run_postprocess_once()
            return [f.value() for f in done.value()]

        return torch.futures.collect_all(futs).then(_then)

    def result(self):
        self.wait()
        return [w.result() for w in self.works]
